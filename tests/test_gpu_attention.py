"""GPU parity of the single-token attention, the embedding look-up and the arg-max against the golden vectors
generated from the reference and against the NumPy oracle."""
import numpy as np
import pytest

from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FA, FW = 16, 24


def _run(q, ck, cv, pos, H, Hkv, hd, window, rope=0, cos=None, sin=None, rows=None):
    """Feeds the cache rows 0..pos-1, then calls the entry for the token at `pos` with un-rotated q/k."""
    import torch

    from integer_inference_engine_b200 import device
    rows = rows or pos + 3
    kc = torch.zeros((Hkv, rows, hd), dtype=torch.int32, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:, :pos] = torch.from_numpy(ck[:, :pos].astype(np.int32)).cuda()
    vc[:, :pos] = torch.from_numpy(cv[:, :pos].astype(np.int32)).cuda()
    qd = torch.from_numpy(q.reshape(-1).copy()).cuda()
    kd = torch.from_numpy(ck[:, pos].reshape(-1).copy()).cuda()
    vd = torch.from_numpy(cv[:, pos].reshape(-1).copy()).cuda()
    out = device.attention_decode(qd, kd, vd, kc, vc, pos, H, Hkv, hd, FA, window or 0,
                                  None if cos is None else torch.from_numpy(cos).cuda(),
                                  None if sin is None else torch.from_numpy(sin).cuda(), rope)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    return out.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), qd.cpu().numpy()


@pytest.mark.parametrize("name,Lc,window", [("dec_full", 37, None), ("dec_win", 37, 9)])
def test_golden_decode_cases(golden_dir, name, Lc, window):
    """Same seeds as tests/golden/make_golden.py::attention_fixture (reference: cohere2.attention_cached)."""
    g = np.load(golden_dir / "attention.npz")
    H, Hkv, hd = 4, 2, 16
    r2 = np.random.default_rng(710 + len(name) + Lc)
    q = r2.integers(-(1 << 19), 1 << 19, size=(1, H, hd), dtype=np.int64)
    ck = r2.integers(-(1 << 19), 1 << 19, size=(Hkv, Lc, hd), dtype=np.int64)
    cv = r2.integers(-(1 << 19), 1 << 19, size=(Hkv, Lc, hd), dtype=np.int64)
    # head_dim 16 is below the kernel's 32-lane split: embed each head in 32 columns of zeros (dot products,
    # and therefore every byte of the result, are unchanged; inv_sqrt stays that of head_dim 16)
    import torch

    from integer_inference_engine_b200 import device
    pad = lambda a: np.concatenate([a, np.zeros(a.shape[:-1] + (16,), np.int64)], axis=-1)
    qp, ckp, cvp = pad(q), pad(ck), pad(cv)
    pos = Lc - 1
    kc = torch.zeros((Hkv, Lc + 2, 32), dtype=torch.int32, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:, :pos] = torch.from_numpy(ckp[:, :pos].astype(np.int32)).cuda()
    vc[:, :pos] = torch.from_numpy(cvp[:, :pos].astype(np.int32)).cuda()
    out = device.attention_decode(torch.from_numpy(qp.reshape(-1).copy()).cuda(), torch.from_numpy(ckp[:, pos].reshape(-1).copy()).cuda(),
                                  torch.from_numpy(cvp[:, pos].reshape(-1).copy()).cuda(), kc, vc, pos, H, Hkv, 32, FA, window or 0,
                                  inv_sqrt=int(round((1.0 / 16 ** 0.5) * (1 << FA))))
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(out.cpu().numpy().reshape(H, 32)[:, :16].reshape(1, -1), g[f"att_{name}"])


@pytest.mark.parametrize("H,Hkv,hd,pos,window,rope", [(32, 4, 128, 200, None, 0), (32, 4, 128, 333, 100, 1), (8, 8, 64, 70, None, 2),
                                                     (32, 8, 128, 0, None, 2), (16, 2, 128, 1100, 1024, 1)])
def test_decode_attention_matches_the_oracle(H, Hkv, hd, pos, window, rope):
    rng = np.random.default_rng(H * 7 + pos)
    Lc = pos + 1
    q = rng.integers(-(1 << 20), 1 << 20, size=(1, H, hd), dtype=np.int64)
    k_new = rng.integers(-(1 << 20), 1 << 20, size=(Hkv, 1, hd), dtype=np.int64)
    ck = rng.integers(-(1 << 20), 1 << 20, size=(Hkv, Lc, hd), dtype=np.int64)       # rows < pos: already rotated keys
    cv = rng.integers(-(1 << 20), 1 << 20, size=(Hkv, Lc, hd), dtype=np.int64)
    cos = sin = None
    q_rot, k_rot = q, k_new
    if rope:
        cos, sin = o.build_rope_tables(Lc, hd, 50000.0, FA)
        at = lambda x: o.rope_fixed(x, cos[pos:pos + 1], sin[pos:pos + 1], FA, neox=rope == 2)
        q_rot = at(np.transpose(q, (1, 0, 2))).transpose(1, 0, 2)                     # [H,1,hd] rotated at `pos`
        k_rot = at(k_new)
    ck_full = ck.copy(); ck_full[:, pos:pos + 1] = k_rot
    want = o.attention_cached(q_rot, ck_full, cv, pos, H, Hkv, FA, window)
    ck_in = ck.copy(); ck_in[:, pos:pos + 1] = k_new                                   # the entry rotates the new key itself
    got, kc, vc, q_after = _run(q, ck_in, cv, pos, H, Hkv, hd, window, rope, cos, sin)
    assert np.array_equal(q_after.reshape(1, H, hd), q)                               # the caller's q is left as it was
    assert np.array_equal(kc[:, pos], k_rot[:, 0].astype(np.int32)) and np.array_equal(vc[:, pos], cv[:, pos].astype(np.int32))
    assert np.array_equal(got.reshape(1, -1), want)


def test_cache_overflow_is_flagged():
    import torch

    from integer_inference_engine_b200 import device
    H, Hkv, hd = 4, 2, 32
    q = torch.ones(H * hd, dtype=torch.int64, device="cuda")
    k = torch.ones(Hkv * hd, dtype=torch.int64, device="cuda"); k[3] = 1 << 33
    v = torch.ones(Hkv * hd, dtype=torch.int64, device="cuda")
    kc = torch.zeros((Hkv, 4, hd), dtype=torch.int32, device="cuda"); vc = torch.zeros_like(kc)
    device.attention_decode(q, k, v, kc, vc, 0, H, Hkv, hd, FA)
    torch.cuda.synchronize()
    assert device.read_flags() & 4


def test_embedding_row_and_argmax():
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    rng = np.random.default_rng(5)
    for qt, synth in ((o.Q6_K, o.synth_q6k), (o.Q4_K, o.synth_q4k)):
        raw = synth(rng, 50, 3)
        h = qk.register_weight(raw, 50, 3, qt)
        table = o.dequant(raw, 50, 3, qt, FA)
        for tok in (0, 17, 49):
            assert np.array_equal(device.embed(h, tok, 768, FA).cpu().numpy()[0], table[tok])
        tok_dev = torch.tensor([33], dtype=torch.int32, device="cuda")
        assert np.array_equal(device.embed(h, tok_dev, 768, FA).cpu().numpy()[0], table[33])
    x = rng.integers(-1000, 1000, size=151936, dtype=np.int64)
    x[[7, 90000, 151935]] = 5000
    assert int(device.argmax(torch.from_numpy(x).cuda()).item()) == 7
    x[:] = -5
    assert int(device.argmax(torch.from_numpy(x).cuda()).item()) == 0
    # the batched forms: several rows / several sequences in one launch each
    toks = torch.tensor([49, 0, 17, 17, 33], dtype=torch.int32, device="cuda")
    assert np.array_equal(device.embed_rows(h, toks, 768, FA).cpu().numpy(), table[[49, 0, 17, 17, 33]])
    for n in (151936, 1001, 7):
        xs = rng.integers(-1000, 1000, size=(5, n), dtype=np.int64)
        xs[1, [3, n - 1]] = 7000; xs[2, :] = -9; xs[3, n - 1] = 9000; xs[4, n // 2] = 8000
        want = [int(np.flatnonzero(r == r.max())[0]) for r in xs]
        assert device.argmax_rows(torch.from_numpy(xs).cuda()).cpu().tolist() == want


@pytest.mark.parametrize("form", [0, 1])
def test_every_launch_form_gives_the_same_bytes(form):
    """Three launches and one cooperative launch."""
    from integer_inference_engine_b200 import qk_cuda as qk
    lib = qk.load_library()
    H, Hkv, hd, pos, window = 32, 4, 128, 700, 512
    rng = np.random.default_rng(99)
    Lc = pos + 1
    q = rng.integers(-(1 << 20), 1 << 20, size=(1, H, hd), dtype=np.int64)
    ck = rng.integers(-(1 << 20), 1 << 20, size=(Hkv, Lc, hd), dtype=np.int64)
    cv = rng.integers(-(1 << 20), 1 << 20, size=(Hkv, Lc, hd), dtype=np.int64)
    cos, sin = o.build_rope_tables(Lc, hd, 50000.0, FA)
    at = lambda x: o.rope_fixed(x, cos[pos:pos + 1], sin[pos:pos + 1], FA)
    ck_full = ck.copy(); ck_full[:, pos:pos + 1] = at(ck[:, pos:pos + 1])
    want = o.attention_cached(at(np.transpose(q, (1, 0, 2))).transpose(1, 0, 2), ck_full, cv, pos, H, Hkv, FA, window)
    try:
        lib.iie_set_attn_fused(form)
        for _ in range(2):
            got, _, _, _ = _run(q, ck, cv, pos, H, Hkv, hd, window, 1, cos, sin)
            assert np.array_equal(got.reshape(1, -1), want)
    finally:
        lib.iie_set_attn_fused(1)


@pytest.mark.parametrize(("H", "Hkv", "hd", "start", "m", "window", "rope"),
                         [(4, 2, 64, 0, 12, None, 0), (4, 2, 64, 15, 5, 7, 1), (8, 1, 128, 3, 70, None, 2), (8, 2, 32, 60, 9, 64, 1),
                          (16, 1, 64, 0, 130, 50, 2), (8, 2, 128, 37, 150, 64, 2), (8, 1, 64, 130, 97, None, 1), (32, 4, 128, 100, 90, None, 1),
                          (6, 2, 128, 0, 33, 16, 0)])
def test_prefill_attention_matches_the_checker(H, Hkv, hd, start, m, window, rope):
    """m new tokens at once (causal, optional window, both rotations) against the CPU checker's cached attention."""
    import torch

    from integer_inference_engine_b200 import device
    rng = np.random.default_rng(900 + H + m)
    rows = start + m + 3
    cos, sin = o.build_rope_tables(rows, hd, 50000.0, FA)
    ck = rng.integers(-(1 << 18), 1 << 18, size=(Hkv, rows, hd), dtype=np.int64)
    cv = rng.integers(-(1 << 18), 1 << 18, size=(Hkv, rows, hd), dtype=np.int64)
    q = rng.integers(-(1 << 19), 1 << 19, size=(m, H, hd), dtype=np.int64)
    k = rng.integers(-(1 << 18), 1 << 18, size=(m, Hkv, hd), dtype=np.int64)
    v = rng.integers(-(1 << 18), 1 << 18, size=(m, Hkv, hd), dtype=np.int64)
    qr, kr = q, k
    if rope:
        rot = lambda t: o.rope_fixed(np.transpose(t, (1, 0, 2)), cos[start:start + m], sin[start:start + m], FA,
                                     neox=(rope == 2)).transpose(1, 0, 2)
        qr, kr = rot(q), rot(k)
    want_k, want_v = ck.copy(), cv.copy()
    want_k[:, start:start + m] = np.transpose(kr, (1, 0, 2))
    want_v[:, start:start + m] = np.transpose(v, (1, 0, 2))
    want = o.attention_cached(qr, want_k[:, :start + m], want_v[:, :start + m], start, H, Hkv, FA, window)
    cuda = lambda a, dt=torch.int64: torch.from_numpy(np.ascontiguousarray(a)).to(dt).cuda()
    kc, vc = cuda(ck, torch.int32), cuda(cv, torch.int32)
    device.read_flags()
    got = device.attention_prefill(cuda(q.reshape(m, -1)), cuda(k.reshape(m, -1)), cuda(v.reshape(m, -1)), kc, vc, start, H, Hkv, hd,
                                   FA, window or 0, cuda(cos), cuda(sin), rope)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(kc.cpu().numpy(), want_k) and np.array_equal(vc.cpu().numpy(), want_v)
    # a decode step after the prefill continues from the same cache
    q1 = rng.integers(-(1 << 19), 1 << 19, size=(1, H, hd), dtype=np.int64)
    k1 = rng.integers(-(1 << 18), 1 << 18, size=(1, Hkv, hd), dtype=np.int64)
    v1 = rng.integers(-(1 << 18), 1 << 18, size=(1, Hkv, hd), dtype=np.int64)
    pos = start + m
    got1 = device.attention_decode(cuda(q1.reshape(-1)), cuda(k1.reshape(-1)), cuda(v1.reshape(-1)), kc, vc, pos, H, Hkv, hd, FA,
                                   window or 0, cuda(cos), cuda(sin), rope)
    q1r, k1r = q1, k1
    if rope:
        rot1 = lambda t: o.rope_fixed(np.transpose(t, (1, 0, 2)), cos[pos:pos + 1], sin[pos:pos + 1], FA,
                                      neox=(rope == 2)).transpose(1, 0, 2)
        q1r, k1r = rot1(q1), rot1(k1)
    want_k[:, pos] = k1r[0]; want_v[:, pos] = v1[0]
    want1 = o.attention_cached(q1r, want_k[:, :pos + 1], want_v[:, :pos + 1], pos, H, Hkv, FA, window)
    assert np.array_equal(got1.cpu().numpy().reshape(1, -1), want1)


@pytest.mark.parametrize("qbits", [19, 40])
def test_prefill_tiles_equal_the_per_token_kernels(qbits):
    """A longer prefill (several key chunks, a window that cuts through them, a ragged last tile) through the sixteen-token
    tiles and through the per-token kernels: the same bytes.  qbits = 40 puts query values beyond int32 (the scalar path)."""
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    H, Hkv, hd, start, m, window = 16, 2, 128, 45, 311, 200
    rng = np.random.default_rng(77 + qbits)
    rows = start + m + 1
    cos, sin = o.build_rope_tables(rows, hd, 50000.0, FA)
    cuda = lambda a, dt=torch.int64: torch.from_numpy(np.ascontiguousarray(a)).to(dt).cuda()
    ck = rng.integers(-(1 << 20), 1 << 20, size=(Hkv, rows, hd), dtype=np.int64)
    cv = rng.integers(-(1 << 30), 1 << 30, size=(Hkv, rows, hd), dtype=np.int64)
    q = rng.integers(-(1 << qbits), 1 << qbits, size=(m, H * hd), dtype=np.int64)
    k = rng.integers(-(1 << 20), 1 << 20, size=(m, Hkv * hd), dtype=np.int64)
    v = rng.integers(-(1 << 30), 1 << 30, size=(m, Hkv * hd), dtype=np.int64)
    lib = qk._lib()
    outs = []
    try:
        for form, tile_tc in ((1, 1), (1, 0), (0, 1)):           # tcgen05 tiles, mma.sync tiles, per-token kernels
            lib.iie_set_attn_fused(form); lib.iie_set_attn_tile_tc(tile_tc)
            kc, vc = cuda(ck, torch.int32), cuda(cv, torch.int32)
            got = device.attention_prefill(cuda(q), cuda(k), cuda(v), kc, vc, start, H, Hkv, hd, FA, window, cuda(cos), cuda(sin), 1)
            torch.cuda.synchronize()
            outs.append((got.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy()))
    finally:
        lib.iie_set_attn_fused(1); lib.iie_set_attn_tile_tc(1)
    assert device.read_flags() == 0
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert np.array_equal(a, b)
