"""One GPU rank of the expert-parallel NCCL test (launched by test_gpu_ep.py): builds its expert shard,
runs the exchange and checks its rows against the CPU checker."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
FA, FW = 16, 24


def main():
    rank, world, port, t_per, out_path = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    from integer_inference_engine_b200 import device, ep, qk_cuda as qk
    from oracle import native as onat
    from oracle import qk_oracle as o
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    d, eff, E, k = 512, 256, 8, 3
    T = t_per * world
    router, gate, up, down, h = o.synth_moe(91 + t_per, d, eff, E, T)
    ids_ref, gates_ref, out_ref = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, h, d, eff, FA, FW)
    epr = E // world
    sl = slice(rank * epr, (rank + 1) * epr)
    rh = qk.register_weight(router, E, d // 256, o.Q4_K)
    shard = device.MoELayer(-1, [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in gate[sl]],
                            [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in up[sl]],
                            [qk.register_weight(w, d, eff // 256, o.Q6_K) for w in down[sl]], k, d, eff)
    moe = ep.from_device_layer(rh, shard, E, FA, FW)
    rows = slice(rank * t_per, (rank + 1) * t_per)
    x = torch.from_numpy(h[rows].copy()).cuda()
    ok = True
    for _ in range(2):                                     # twice: workspaces are reused on the second pass
        out, ids, gates = moe.forward(x)
        torch.cuda.synchronize()
        ok = ok and np.array_equal(out.cpu().numpy(), out_ref[rows]) and np.array_equal(ids.cpu().numpy(), ids_ref[rows])
        ok = ok and np.array_equal(gates.cpu().numpy(), gates_ref[rows]) and device.read_flags() == 0
    np.savez(out_path, ok=ok)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
