"""GPU tests of the expert-parallel form of the MoE block: the split entry points on one GPU (two shards
emulated side by side, no collective), and the NCCL exchange on two GPUs when the box has them."""
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import native as onat
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FA, FW = 16, 24
HERE = Path(__file__).resolve().parent


@pytest.mark.parametrize("d,eff,E,k,T,shards", [(512, 256, 8, 2, 5, 2), (2048, 768, 16, 8, 1, 4), (256, 256, 8, 3, 260, 2)])
def test_route_and_sharded_expert_stage_equal_the_block(d, eff, E, k, T, shards):
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    qk.free_all()
    router, gate, up, down, h = o.synth_moe(70 + d + T, d, eff, E, T)
    ids_ref, gates_ref, out_ref = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, h, d, eff, FA, FW)
    rh = qk.register_weight(router, E, d // 256, o.Q4_K)
    x = torch.from_numpy(h).cuda()
    ids, gates = device.route(rh, k, x, FA, FW)
    assert np.array_equal(ids.cpu().numpy(), ids_ref) and np.array_equal(gates.cpu().numpy(), gates_ref)
    epr = E // shards
    total = torch.zeros_like(x)
    for s in range(shards):
        sl = slice(s * epr, (s + 1) * epr)
        layer = device.MoELayer(-1, [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in gate[sl]],
                                [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in up[sl]],
                                [qk.register_weight(w, d, eff // 256, o.Q6_K) for w in down[sl]], k, d, eff)
        part = layer.experts(x, ids, gates, s * epr, FA, FW)
        total += part
        with pytest.raises(qk.CudaContextError):
            layer.forward(x, FA, FW)                      # a shard without a router cannot run the whole block
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(total.cpu().numpy(), out_ref)


def _wait_all(procs, timeout):
    """Wait for every rank; as soon as one fails or the time runs out, the others are killed, so that no rank is
    left inside a collective holding a device."""
    import time
    deadline = time.monotonic() + timeout
    try:
        pending = list(procs)
        while pending:
            for p in list(pending):
                rc = p.poll()
                if rc is None:
                    continue
                pending.remove(p)
                assert rc == 0, f"rank process exited with {rc}"
            assert time.monotonic() < deadline, "rank processes timed out"
            time.sleep(0.05)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
            p.wait()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("T_per_rank", [1, 8])
def test_nccl_exchange_on_two_gpus(T_per_rank, tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, str(HERE / "ep_gpu_worker.py"), str(r), "2", str(port), str(T_per_rank),
                               str(tmp_path / f"r{r}.npz")]) for r in range(2)]
    _wait_all(procs, 240)
    parts = [np.load(tmp_path / f"r{r}.npz") for r in range(2)]
    assert all(bool(p["ok"]) for p in parts)
