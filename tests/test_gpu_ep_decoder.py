"""GPU tests of the expert-parallel batched decode: batched attention over independent sequences against the CPU checker,
the one-rank decoder against the per-sequence checker of a whole decode step, and (on a box with two GPUs) byte identity of
the two-rank run with the one-rank run."""
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import model_oracle
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FA, FW = 16, 24
HERE = Path(__file__).resolve().parent


@pytest.mark.parametrize(("B", "H", "Hkv", "hd", "pos", "window", "rope", "kbits"),
                         [(3, 4, 2, 64, 20, None, 0, 19), (5, 8, 2, 64, 37, 9, 1, 19), (2, 8, 1, 128, 130, 64, 1, 19),
                          # long enough for several CTAs to share one pair's key chunks
                          (2, 8, 2, 64, 700, None, 1, 19), (3, 16, 2, 128, 450, 300, 0, 19),
                          # cached keys beyond 24 bits in some chunks only: the four-plane and the three-plane products side by side
                          (2, 8, 2, 64, 300, None, 1, 29), (2, 8, 1, 128, 200, None, 0, 30)])
def test_batched_decode_attention_matches_the_checker_per_sequence(B, H, Hkv, hd, pos, window, rope, kbits):
    import torch

    from integer_inference_engine_b200 import device
    rng = np.random.default_rng(B * 100 + pos)
    rows = pos + 3
    q = rng.integers(-(1 << 19), 1 << 19, size=(B, H * hd), dtype=np.int64)
    k = rng.integers(-(1 << 19), 1 << 19, size=(B, Hkv * hd), dtype=np.int64)
    v = rng.integers(-(1 << 19), 1 << 19, size=(B, Hkv * hd), dtype=np.int64)
    kc = rng.integers(-(1 << 19), 1 << 19, size=(B, Hkv, rows, hd)).astype(np.int32)
    if kbits > 19:
        kc[:, :, 70:190] = rng.integers(-(1 << kbits), 1 << kbits, size=(B, Hkv, 120, hd)).astype(np.int32)
    vc = rng.integers(-(1 << 19), 1 << 19, size=(B, Hkv, rows, hd)).astype(np.int32)
    cos, sin = o.build_rope_tables(rows, hd, 50000.0, FA)
    kcd, vcd = torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda()
    got = device.attention_decode_batch(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), kcd, vcd, pos,
                                        H, Hkv, hd, FA, window or 0, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), rope)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    rot = (lambda t: o.rope_fixed(t, cos[pos:pos + 1], sin[pos:pos + 1], FA)) if rope else (lambda t: t)
    for b in range(B):
        qb = rot(q[b].reshape(H, 1, hd)).transpose(1, 0, 2)
        kb = rot(k[b].reshape(Hkv, 1, hd))
        ck, cv = kc[b].astype(np.int64)[:, :pos + 1].copy(), vc[b].astype(np.int64)[:, :pos + 1].copy()
        ck[:, pos] = kb[:, 0]; cv[:, pos] = v[b].reshape(Hkv, hd)
        want = o.attention_cached(qb, ck, cv, pos, H, Hkv, FA, window)
        assert np.array_equal(got[b].cpu().numpy(), want[0]), b
        assert np.array_equal(kcd[b, :, pos].cpu().numpy(), ck[:, pos].astype(np.int32))      # the appended rows
        assert np.array_equal(vcd[b, :, pos].cpu().numpy(), cv[:, pos].astype(np.int32))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(world, n_seqs, tmp_path, tag, timeout=150):
    """Start one process per rank; poll them all, and as soon as one fails or the time runs out kill the others, so that no
    rank is left waiting inside a collective.  The ranks' output goes to files whose tails are shown on failure."""
    import time
    port = _free_port()
    logs = [open(tmp_path / f"{tag}{r}.log", "w") for r in range(world)]
    procs = [subprocess.Popen([sys.executable, str(HERE / "ep_decoder_worker.py"), str(r), str(world), str(port), str(n_seqs),
                               str(tmp_path / f"{tag}{r}.npz")], stdout=logs[r], stderr=subprocess.STDOUT) for r in range(world)]
    deadline, failed = time.monotonic() + timeout, None
    try:
        pending = list(range(world))
        while pending and failed is None:
            for r in list(pending):
                rc = procs[r].poll()
                if rc is not None:
                    pending.remove(r)
                    if rc != 0:
                        failed = f"rank {r} exited with {rc}"
            if failed is None and pending and time.monotonic() > deadline:
                failed = f"ranks {pending} still running after {timeout} s"
            time.sleep(0.05)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
            p.wait()
        for f in logs:
            f.close()
    if failed:
        tails = "\n".join(f"--- rank {r} ---\n" + (tmp_path / f"{tag}{r}.log").read_text()[-1500:] for r in range(world))
        raise AssertionError(f"{failed}\n{tails}")
    return [np.load(tmp_path / f"{tag}{r}.npz") for r in range(world)]


def test_one_rank_decoder_matches_the_checker_for_every_sequence(tmp_path):
    """Every sequence of the batched one-rank decoder equals the per-sequence CPU checker of a whole decode step."""
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    from integer_inference_engine_b200.ep_model import ExpertParallelDecoder
    from tests.ep_decoder_worker import SHAPE
    qk.free_all()
    m = ExpertParallelDecoder(3, **SHAPE)
    nb, E, eff = m.d // 256, SHAPE["n_experts"], SHAPE["e_ffn"]
    qr, kr = m.H * m.hd, m.Hkv * m.hd
    host = []
    for li in range(m.n_layers):
        a, hs = m.attn[li], m.stack.handles[li]
        fused = device.export_weight(a["wqkv"], qr + 2 * kr, nb, o.Q4_K)
        cut = lambda r0, r1: bytes(fused[r0 * nb * 144:r1 * nb * 144])
        host.append({"gain": hs["gain"].cpu().numpy(), "wq": cut(0, qr), "wk": cut(qr, qr + kr), "wv": cut(qr + kr, qr + 2 * kr),
                     "wo": device.export_weight(a["wo"], m.d, qr // 256, o.Q4_K), "full": m.layer_is_full(li),
                     "moe": (device.export_weight(hs["router"], E, nb, o.Q4_K),
                             [device.export_weight(x, eff, nb, o.Q4_K) for x in hs["gate"]],
                             [device.export_weight(x, eff, nb, o.Q4_K) for x in hs["up"]],
                             [device.export_weight(x, m.d, eff // 256, o.Q6_K) for x in hs["down"]]),
                     "kall": a["k"].cpu().numpy().astype(np.int64), "vall": a["v"].cpu().numpy().astype(np.int64)})
    embd = device.export_weight(m.embd, m.vocab, nb, o.Q6_K)
    cfg = dict(d=m.d, H=m.H, Hkv=m.Hkv, hd=m.hd, eff=eff, E=E, k=m.top_k, vocab=m.vocab, window=m.window, fa=FA, fw=FW)
    first = np.array([3, 10, 17], dtype=np.int32)
    m.tokens.copy_(torch.from_numpy(first).cuda())
    m.step()
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    for b in range(3):
        layers = [dict(L, k=L["kall"][b].copy(), v=L["vall"][b].copy()) for L in host]
        want, trace, _ = model_oracle.decode_token(int(first[b]), m.position, layers, embd, m.out_gain.cpu().numpy(), cfg,
                                                   m.cos.cpu().numpy(), m.sin.cpu().numpy())
        assert np.array_equal(m.x[b].cpu().numpy(), trace[-1]), b
        assert int(m.tokens[b].item()) == want
    qk.free_all()


def test_two_ranks_reproduce_one_rank_bytes(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    one = _run_ranks(1, 4, tmp_path, "one")[0]
    two = _run_ranks(2, 4, tmp_path, "two")
    assert bool(one["ok"]) and all(bool(p["ok"]) for p in two)
    for key in ("t1", "x1", "t2", "x2", "k0"):
        assert np.array_equal(np.concatenate([p[key] for p in two]), one[key]), key
