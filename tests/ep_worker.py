"""One CPU rank of the expert-parallel exchange test (launched by test_ep_cpu.py; gloo backend).

The two compute steps of ExpertParallelMoE are filled with the NumPy checker, so what runs here is the
host-side exchange logic: segment packing, both all-to-alls, the skip of foreign slots, the combine order."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
from integer_inference_engine_b200.ep import ExpertParallelMoE   # noqa: E402
from oracle import qk_oracle as o   # noqa: E402

FA, FW = 16, 24


def main():
    rank, world, port, out_path = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    seed, d, eff, E, k, T = o.GOLDEN_MOE_CASES["small"]
    router, gate, up, down, h = o.synth_moe(seed, d, eff, E, T)
    rw = o.dequant(router, E, d // 256, o.Q4_K, FW)
    epr = E // world
    mine = {e: (o.dequant(gate[e], eff, d // 256, o.Q4_K, FW), o.dequant(up[e], eff, d // 256, o.Q4_K, FW),
                o.dequant(down[e], d, eff // 256, o.Q6_K, FW)) for e in range(rank * epr, (rank + 1) * epr)}

    def route_fn(x):
        _, ids, gates = o.route(x.numpy(), rw, k, FA, FW)
        return torch.from_numpy(ids), torch.from_numpy(gates)

    def experts_fn(rows, ids, gates, base):
        assert base == rank * epr
        rows, ids, gates = rows.numpy(), ids.numpy(), gates.numpy()
        out = np.zeros(rows.shape, dtype=object)
        for t in range(rows.shape[0]):
            for j in range(ids.shape[1]):
                e = int(ids[t, j])
                if e in mine:                                       # slots of other shards are skipped
                    eo = o.expert_ffn(rows[t:t + 1], *mine[e], FA, FW).astype(object)
                    out[t] += (eo * int(gates[t, j])) >> FA
        return torch.from_numpy(out.astype(np.int64))

    ep = ExpertParallelMoE(E, k, d, route_fn, experts_fn)
    per = T // world
    x = torch.from_numpy(h[rank * per:(rank + 1) * per].copy())
    out, ids, gates = ep.forward(x)
    np.savez(out_path, out=out.numpy(), ids=ids.numpy(), gates=gates.numpy(), sent=ep.bytes_sent_last)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
