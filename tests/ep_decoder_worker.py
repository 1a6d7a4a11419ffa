"""One rank of the expert-parallel decoder test (launched by test_gpu_ep_decoder.py): builds its share of a small
decoder, runs two lockstep decode steps (the second as a replayed graph) and saves what its sequences produced."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

SHAPE = dict(n_layers=3, d_model=512, n_heads=8, n_kv=2, head_dim=64, e_ffn=256, n_experts=8, top_k=2, vocab=640, context=70,
             max_new=4, window=32, seed=11)


def main():
    import faulthandler
    faulthandler.dump_traceback_later(100, exit=False)      # a rank that hangs leaves its stack in the log the test shows
    rank, world, port, n_seqs, out_path = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    from integer_inference_engine_b200 import device
    from integer_inference_engine_b200.ep_model import ExpertParallelDecoder
    torch.cuda.set_device(rank)
    if world > 1:
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
    m = ExpertParallelDecoder(n_seqs, **SHAPE)
    first = torch.arange(rank * m.B, (rank + 1) * m.B, dtype=torch.int32, device="cuda") * 7 + 3
    m.tokens.copy_(first)
    m.step()                                                # eager
    torch.cuda.synchronize()
    t1, x1 = m.tokens.cpu().numpy().copy(), m.x.cpu().numpy().copy()
    m.advance()
    m.capture()
    m.replay()                                              # the second token as one replayed graph
    torch.cuda.synchronize()
    ok = device.read_flags() == 0
    np.savez(out_path, ok=ok, t1=t1, x1=x1, t2=m.tokens.cpu().numpy(), x2=m.x.cpu().numpy(),
             k0=m.attn[0]["k"][:, :, SHAPE["context"]:SHAPE["context"] + 2].cpu().numpy())
    if world > 1:
        # every rank has saved its results; tearing the process group down while a captured graph still holds collective
        # launches can block, so the graph is released first and the process leaves without the teardown
        dist.barrier()
        torch.cuda.synchronize()
        m._graph = None
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
