"""GPU suite: the CUDA path, called through the C-ABI, is byte-identical to the CPU oracle.

Mirrors the reference's differential tests (north-mini-code/tests/test_qk_cuda.py): fused linear on
odd shapes, resident == per-call, negative floor, RMSNorm + router + top-k incl. the all-equal tie,
fused MoE == per-expert composition, mixed Q4_K/Q6_K experts, batched == per-token, registry
lifecycle, large magnitudes that need more than four limbs, and inputs beyond the limb envelope
(which must take the 128-bit kernel and still match)."""
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

from oracle import native as onat
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu

FA, FW = 16, 24


@pytest.fixture(scope="module")
def qk():
    from integer_inference_engine_b200 import qk_cuda
    assert qk_cuda.available(), "CUDA library or GPU missing: the product path has no fallback"
    yield qk_cuda
    qk_cuda.free_all()


def _synth(rng, qt, out_f, nb):
    return (o.synth_q4k if qt == o.Q4_K else o.synth_q6k)(rng, out_f, nb)


@pytest.mark.parametrize("qtype", [o.Q4_K, o.Q6_K])
@pytest.mark.parametrize("out_f,n_blocks,T", [(8, 1, 1), (16, 2, 3), (5, 3, 4), (64, 8, 2), (262, 8, 1), (1, 1, 1),
                                               (33, 16, 5), (40, 3, 7)])
def test_linear_matches_oracle(qk, qtype, out_f, n_blocks, T):
    rng = np.random.default_rng(out_f + n_blocks + T + qtype)
    raw = _synth(rng, qtype, out_f, n_blocks)
    x = rng.integers(-(1 << (FW - 6)), 1 << (FW - 6), size=(T, n_blocks * 256), dtype=np.int64)
    got = qk.qk_linear(raw, x, out_f, n_blocks, FW, qtype)
    assert got is not None
    assert np.array_equal(got, onat.qk_linear(raw, x, out_f, n_blocks, FW, qtype))
    if out_f * n_blocks * T <= 64:
        assert np.array_equal(got, o.qk_linear(raw, x, out_f, n_blocks, FW, qtype))


@pytest.mark.parametrize("out_f,n_blocks,T,xbits", [(150, 2, 200, 20), (128, 1, 260, 34), (300, 3, 192, 12)])
def test_prefill_sized_linear_runs_on_the_tensor_core_tiles(qk, out_f, n_blocks, T, xbits):
    """From 192 rows on a dense Q4_K product takes the tcgen05 tiles (three or five activation digits); same answer."""
    from integer_inference_engine_b200 import device
    rng = np.random.default_rng(out_f + T)
    raw = _synth(rng, o.Q4_K, out_f, n_blocks)
    x = rng.integers(-(1 << xbits), 1 << xbits, size=(T, n_blocks * 256), dtype=np.int64)
    before = device.prefill_launch_counts()
    got = qk.qk_linear(raw, x, out_f, n_blocks, FW, o.Q4_K)
    delta = [b - a for a, b in zip(before, device.prefill_launch_counts())]
    assert got is not None and np.array_equal(got, onat.qk_linear(raw, x, out_f, n_blocks, FW, o.Q4_K))
    assert delta[5] + delta[6] == 1, f"the product did not reach the tensor-core tiles: {delta}"


def test_linear_golden_vectors(qk, golden_dir):
    g = np.load(golden_dir / "linear.npz")
    for i, (qt, out_f, nb, T, magbits) in enumerate(o.GOLDEN_LINEAR_CASES):
        rng = np.random.default_rng(200 + i)
        raw = _synth(rng, qt, out_f, nb)
        x = rng.integers(-(1 << magbits), 1 << magbits, size=(T, nb * 256), dtype=np.int64)
        assert np.array_equal(qk.qk_linear(raw, x, out_f, nb, FW, qt), g[f"y_{i}"]), i


@pytest.mark.parametrize("qtype", [o.Q4_K, o.Q6_K])
def test_linear_arbitrary_block_bytes(qk, qtype):
    """Any bytes form a valid block: random scales up to the largest finite half, all sub-block
    scale/min patterns.  Large block scales leave the fast envelope and take the 128-bit kernel."""
    rng = np.random.default_rng(77 + qtype)
    out_f, nb, bs = 24, 2, (144 if qtype == o.Q4_K else 210)
    b = rng.integers(0, 256, size=(out_f * nb, bs), dtype=np.uint8)
    for pos in ((1, 3) if qtype == o.Q4_K else (209,)):
        b[:, pos] &= 0x7B                                         # keep the halves finite
    x = rng.integers(-(1 << 20), 1 << 20, size=(2, nb * 256), dtype=np.int64)
    got = qk.qk_linear(b.tobytes(), x, out_f, nb, FW, qtype)
    assert np.array_equal(got, onat.qk_linear(b.tobytes(), x, out_f, nb, FW, qtype))
    b[:, (1 if qtype == o.Q4_K else 209)] &= 0x1F                 # small scales: fast path, same bytes otherwise
    if qtype == o.Q4_K:
        b[:, 3] &= 0x1F
    got = qk.qk_linear(b.tobytes(), x, out_f, nb, FW, qtype)
    assert np.array_equal(got, onat.qk_linear(b.tobytes(), x, out_f, nb, FW, qtype))


@pytest.mark.parametrize("fw", [24, 16, 20, 0])
def test_linear_other_weight_scales(qk, fw):
    """fw below 24 makes half -> fixed round (half to even); the kernel's integer conversion must agree."""
    rng = np.random.default_rng(fw)
    for qt in (o.Q4_K, o.Q6_K):
        raw = _synth(rng, qt, 16, 2)
        x = rng.integers(-(1 << 16), 1 << 16, size=(2, 512), dtype=np.int64)
        assert np.array_equal(qk.qk_linear(raw, x, 16, 2, fw, qt), onat.qk_linear(raw, x, 16, 2, fw, qt))


def test_negative_floor(qk):
    rng = np.random.default_rng(2)
    raw = o.synth_q4k(rng, 4, 4)
    x = -np.abs(rng.integers(1, 1 << 14, size=(2, 1024), dtype=np.int64))
    assert np.array_equal(qk.qk_linear(raw, x, 4, 4, FW, o.Q4_K), o.qk_linear(raw, x, 4, 4, FW, o.Q4_K))


@pytest.mark.parametrize("magbits", [27, 40, 55, 62])
def test_large_magnitudes(qk, magbits):
    """More than four limbs (the reference's dp4a ceiling) stay on the fast path here; values close
    to the int64 range exceed eight balanced digits and must take the exact 128-bit kernel."""
    rng = np.random.default_rng(magbits)
    for qt in (o.Q4_K, o.Q6_K):
        raw = _synth(rng, qt, 24, 2, )
        x = rng.integers(-(1 << magbits), 1 << magbits, size=(3, 512), dtype=np.int64)
        if magbits == 62:
            x[0, 0] = np.iinfo(np.int64).max
            x[1, 5] = np.iinfo(np.int64).min
        assert np.array_equal(qk.qk_linear(raw, x, 24, 2, FW, qt), onat.qk_linear(raw, x, 24, 2, FW, qt))


def test_resident_matches_percall_and_dense_handle_is_rejected(qk):
    qk.free_all()
    rng = np.random.default_rng(7)
    for qt in (o.Q4_K, o.Q6_K):
        out_f, nb, T = 16, 4, 3
        raw = _synth(rng, qt, out_f, nb)
        x = rng.integers(-(1 << 16), 1 << 16, size=(T, nb * 256), dtype=np.int64)
        h = qk.register_weight(raw, out_f, nb, qt)
        got = qk.apply_resident(h, x, out_f, FW)
        assert np.array_equal(got, onat.qk_linear(raw, x, out_f, nb, FW, qt))
        assert np.array_equal(got, qk.qk_linear(raw, x, out_f, nb, FW, qt))
        assert np.array_equal(qk.apply_resident_dp4a(h, x, out_f, FW, qt), got)
        assert qk.apply_resident_dp4a(h, x, out_f, FW, 1 - qt) is None          # wrong type -> rc 2
    dense = qk.register_i64(np.arange(256, dtype=np.int64))
    assert qk.apply_resident(dense, np.zeros((1, 256), np.int64), 1, FW) is None
    assert qk.apply_resident(12345, np.zeros((1, 256), np.int64), 1, FW) is None
    qk.free_all()


def test_grouped_apply_equals_separate_applies(qk):
    qk.free_all()
    rng = np.random.default_rng(17)
    nb, T = 2, 3
    shapes = [(32, o.Q4_K), (8, o.Q4_K), (8, o.Q6_K), (24, o.Q6_K)]
    raws = [_synth(rng, qt, of, nb) for of, qt in shapes]
    hs = [qk.register_weight(r, of, nb, qt) for r, (of, qt) in zip(raws, shapes)]
    x = rng.integers(-(1 << 18), 1 << 18, size=(T, nb * 256), dtype=np.int64)
    got = qk.apply_resident_grouped(hs, x, [of for of, _ in shapes], FW, phase_ids=[1, 2, 3, 4])
    assert got is not None and len(got) == 4
    for y, h, (of, _) in zip(got, hs, shapes):
        assert np.array_equal(y, qk.apply_resident(h, x, of, FW))
    qk.free_all()


def test_rmsnorm_router_topk(qk):
    qk.free_all()
    rng = np.random.default_rng(1907)
    rows, width, experts, used = 3, 256, 8, 3
    x = rng.integers(-(1 << 18), 1 << 18, size=(rows, width), dtype=np.int64)
    gain = rng.integers(1 << 15, 1 << 17, size=width, dtype=np.int64)
    router = rng.integers(-(1 << 13), 1 << 13, size=(experts, width), dtype=np.int64)
    gh, rh = qk.register_i64(gain), qk.register_i64(router)
    h, ids, gates = qk.rmsnorm_router(gh, rh, x, used, FA, FW, eps=1)
    ref_h = o.rmsnorm_fixed(x, FA, 1, gain)
    _, ref_ids, ref_gates = o.route(ref_h, router, used, FA, FW)
    assert np.array_equal(h, ref_h) and np.array_equal(ids, ref_ids) and np.array_equal(gates, ref_gates)
    # equal logits keep ascending expert ids
    zh = qk.register_i64(np.zeros_like(router))
    tied = qk.rmsnorm_router(gh, zh, x[:1], used, FA, FW)
    assert tied[1].tolist() == [list(range(used))]
    assert tied[2].tolist() == [[int(o.sigmoid_fixed(np.array([0]), FA)[0])] * used]
    # a row whose sum of squares leaves 128 bits is declined before any native work
    unsafe = np.zeros((1, width), np.int64)
    unsafe[0, :2] = np.iinfo(np.int64).min
    assert qk.rmsnorm_router(gh, rh, unsafe, used, FA, FW) is None
    qk.free_all()


def test_rmsnorm_router_real_shape(qk):
    qk.free_all()
    rng = np.random.default_rng(5)
    rows, width, experts, used = 4, 2048, 128, 8
    x = o.to_fixed(rng.standard_normal((rows, width)) * 3, FA)
    gain = o.to_fixed(np.abs(rng.standard_normal(width)) + 0.5, FA)
    router = o.to_fixed(rng.standard_normal((experts, width)) * 0.05, FW)
    gh, rh = qk.register_i64(gain), qk.register_i64(router)
    h, ids, gates = qk.rmsnorm_router(gh, rh, x, used, FA, FW)
    ref_h = o.rmsnorm_fixed(x, FA, 1, gain)
    _, ref_ids, ref_gates = o.route(ref_h, router, used, FA, FW)
    assert np.array_equal(h, ref_h) and np.array_equal(ids, ref_ids) and np.array_equal(gates, ref_gates)
    qk.free_all()


def _register_experts(qk, rng, n, d_model, e_ffn, down_qt):
    nb_in, nb_dn = d_model // 256, e_ffn // 256
    raws = {"gate": [o.synth_q4k(rng, e_ffn, nb_in) for _ in range(n)],
            "up": [o.synth_q4k(rng, e_ffn, nb_in) for _ in range(n)],
            "down": [_synth(rng, down_qt, d_model, nb_dn) for _ in range(n)]}
    hs = {"gate": [qk.register_weight(r, e_ffn, nb_in, o.Q4_K) for r in raws["gate"]],
          "up": [qk.register_weight(r, e_ffn, nb_in, o.Q4_K) for r in raws["up"]],
          "down": [qk.register_weight(r, d_model, nb_dn, down_qt) for r in raws["down"]]}
    return raws, hs


def _moe_ref(raws, sel, h, gates, d_model, e_ffn, down_qt):
    ref = np.zeros(d_model, dtype=object)
    for j, e in enumerate(sel):
        g = onat.silu(onat.qk_linear(raws["gate"][e], h[None], e_ffn, d_model // 256, FW, o.Q4_K)[0], FA)
        u = onat.qk_linear(raws["up"][e], h[None], e_ffn, d_model // 256, FW, o.Q4_K)[0]
        gu = o.mul_shift(g, u, FA)
        dn = onat.qk_linear(raws["down"][e], gu[None], d_model, e_ffn // 256, FW, down_qt)[0]
        ref += (dn.astype(object) * int(gates[j])) >> FA
    return ref.astype(np.int64)


@pytest.mark.parametrize("down_qt", [o.Q4_K, o.Q6_K])
def test_moe_ffn_matches_per_expert_composition(qk, down_qt):
    qk.free_all()
    rng = np.random.default_rng(11)
    n_e, d_model, e_ffn = 4, 512, 256
    raws, hs = _register_experts(qk, rng, n_e, d_model, e_ffn, down_qt)
    h = rng.integers(-(1 << 16), 1 << 16, size=d_model, dtype=np.int64)
    gates = rng.integers(0, 1 << 16, size=n_e, dtype=np.int64)
    got = qk.moe_ffn(hs["gate"], hs["up"], hs["down"], h, gates, d_model, e_ffn, FA, FW)
    grows = qk.moe_workspace_allocations()
    again = qk.moe_ffn(hs["gate"], hs["up"], hs["down"], h, gates, d_model, e_ffn, FA, FW, dp4a=True)
    assert np.array_equal(again, got)
    assert grows > 0 and qk.moe_workspace_allocations() == grows        # steady state allocates nothing
    assert np.array_equal(got, _moe_ref(raws, range(n_e), h, gates, d_model, e_ffn, down_qt))
    with ThreadPoolExecutor(max_workers=4) as pool:                         # callers are serialised, results identical
        results = list(pool.map(lambda _: qk.moe_ffn(hs["gate"], hs["up"], hs["down"], h, gates, d_model, e_ffn, FA, FW),
                                range(8)))
    assert all(np.array_equal(r, got) for r in results)
    qk.free_all()


def test_moe_ffn_outside_the_limb_envelope_uses_the_exact_kernels(qk):
    """A hidden state needing a ninth digit, and a gate*up product that does, both still match."""
    qk.free_all()
    rng = np.random.default_rng(12)
    n_e, d_model, e_ffn = 2, 256, 256
    raws, hs = _register_experts(qk, rng, n_e, d_model, e_ffn, o.Q6_K)
    gates = rng.integers(0, 1 << 16, size=n_e, dtype=np.int64)
    h = rng.integers(-(1 << 10), 1 << 10, size=d_model, dtype=np.int64)
    h[3] = qk._balanced_capacity(8) + 5
    got = qk.moe_ffn(hs["gate"], hs["up"], hs["down"], h, gates, d_model, e_ffn, FA, FW)
    def wrap_ref():
        # expected value with the reference's two's-complement truncation of each 128-bit result
        ref = np.zeros(d_model, dtype=np.uint64)
        for j in range(n_e):
            g = onat.qk_linear(raws["gate"][j], h[None], e_ffn, 1, FW, o.Q4_K)[0]
            u = onat.qk_linear(raws["up"][j], h[None], e_ffn, 1, FW, o.Q4_K)[0]
            sg = onat.sigmoid(g, FA)
            s = np.array([((int(a) * int(b)) >> FA) for a, b in zip(g, sg)], dtype=object)
            gu = np.array([(((int(a) * int(b)) >> FA) + (1 << 63)) % (1 << 64) - (1 << 63) for a, b in zip(s, u)], dtype=np.int64)
            dn = onat.qk_linear(raws["down"][j], gu[None], d_model, 1, FW, o.Q6_K)[0]
            term = np.array([(((int(a) * int(gates[j])) >> FA)) % (1 << 64) for a in dn], dtype=np.uint64)
            ref += term
        return ref.view(np.int64)
    assert np.array_equal(got, wrap_ref())
    qk.free_all()


def test_moe_ffn_batched_matches_per_token(qk):
    qk.free_all()
    rng = np.random.default_rng(21)
    n_pool, m, k, d_model, e_ffn = 6, 5, 2, 512, 256
    raws, hs = _register_experts(qk, rng, n_pool, d_model, e_ffn, o.Q6_K)
    h = rng.integers(-(1 << 16), 1 << 16, size=(m, d_model), dtype=np.int64)
    sel = [rng.choice(n_pool, k, replace=False) for _ in range(m)]
    gts = [rng.integers(0, 1 << 16, size=k).astype(np.int64) for _ in range(m)]
    flat = lambda name: [hs[name][e] for t in range(m) for e in sel[t]]
    gflat = [int(g) for t in range(m) for g in gts[t]]
    got = qk.moe_ffn_batched(flat("gate"), flat("up"), flat("down"), m, k, h, gflat, d_model, e_ffn, FA, FW)
    grows = qk.moe_workspace_allocations()
    again = qk.moe_ffn_batched(flat("gate"), flat("up"), flat("down"), m, k, h, gflat, d_model, e_ffn, FA, FW, dp4a=True)
    assert np.array_equal(again, got) and qk.moe_workspace_allocations() == grows
    for t in range(m):
        assert np.array_equal(got[t], _moe_ref(raws, sel[t], h[t], gts[t], d_model, e_ffn, o.Q6_K)), t
        one = qk.moe_ffn([hs["gate"][e] for e in sel[t]], [hs["up"][e] for e in sel[t]], [hs["down"][e] for e in sel[t]],
                         h[t], gts[t], d_model, e_ffn, FA, FW)
        assert np.array_equal(got[t], one)
    kept = qk.resident_count()
    assert qk.moe_workspace_bytes() > 0 and qk.release_moe_workspace() and qk.moe_workspace_bytes() == 0
    assert qk.resident_count() == kept
    assert np.array_equal(qk.moe_ffn_batched(flat("gate"), flat("up"), flat("down"), m, k, h, gflat, d_model, e_ffn, FA, FW), got)
    qk.free_all()


def test_registry_lifecycle_and_profile_counters(qk):
    qk.free_all()
    assert qk.reserve_resident_capacity(16_385) and qk.resident_capacity() >= 16_385 and qk.resident_count() == 0
    rng = np.random.default_rng(991)
    raw = o.synth_q6k(rng, 8, 4)
    x = rng.integers(-(1 << 16), 1 << 16, size=(1, 1024), dtype=np.int64)
    h1 = qk.register_weight(raw, 8, 4, o.Q6_K)
    r1 = qk.apply_resident(h1, x, 8, FW)
    qk.free_all()
    assert qk.resident_capacity() == 0 and qk.resident_count() == 0
    assert qk.profile_reset(enabled=True)
    h2 = qk.register_weight(raw, 8, 4, o.Q6_K)
    r2 = qk.apply_resident(h2, x, 8, FW)
    assert np.array_equal(r1, r2)
    stats = qk.profile_snapshot()
    assert stats["native_calls"] == 2 and stats["resident_apply_calls"] == 1 and stats["registration_calls"] == 1
    assert stats["h2d_bytes"] >= len(raw) + x.nbytes and stats["d2h_bytes"] >= r2.nbytes
    qk.profile_set_enabled(False)
    qk.free_all()


# ------------------------------------------------------------------------------------------------
# device-tensor front end: the fused single-token path (routing kernel + streamed gate/up + down)
# and the batched dispatch path, against the C oracle
# ------------------------------------------------------------------------------------------------
def _device_layer(qk, seed, d, eff, E, k, T, xbits=None):
    import torch

    from integer_inference_engine_b200 import device
    router, gate, up, down, h = o.synth_moe(seed, d, eff, E, T)
    if xbits is not None:
        h = np.random.default_rng(seed).integers(-(1 << xbits), 1 << xbits, size=(T, d), dtype=np.int64)
    rh = qk.register_weight(router, E, d // 256, o.Q4_K)
    gh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in gate]
    uh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in up]
    dh = [qk.register_weight(w, d, eff // 256, o.Q6_K) for w in down]
    layer = device.MoELayer(rh, gh, uh, dh, k, d, eff)
    ref = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, h, d, eff, FA, FW)
    return layer, torch.from_numpy(h).cuda(), ref


@pytest.mark.parametrize("d,eff,E,k,T,xbits", [(512, 256, 8, 2, 1, None), (2048, 768, 20, 8, 1, None),
                                              (256, 512, 5, 3, 1, None), (512, 256, 8, 2, 1, 22),
                                              (512, 256, 8, 2, 6, None), (2048, 768, 128, 8, 1, None)])
def test_device_moe_forward(qk, d, eff, E, k, T, xbits):
    import torch

    from integer_inference_engine_b200 import device
    qk.free_all()
    layer, h, (ids_ref, gates_ref, out_ref) = _device_layer(qk, 40 + d + E, d, eff, E, k, T, xbits)
    out, ids, gates = layer.forward(h, FA, FW)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert np.array_equal(gates.cpu().numpy(), gates_ref)
    assert np.array_equal(out.cpu().numpy(), out_ref)
    acc = torch.ones_like(out)                                   # accumulate adds to what is there
    layer.forward(h, FA, FW, out=acc, accumulate=True)
    assert np.array_equal(acc.cpu().numpy(), out_ref + 1)
    qk.free_all()


@pytest.mark.parametrize("T", [1, 3])
def test_device_moe_block_with_norm_and_residual(qk, T):
    import torch

    from integer_inference_engine_b200 import device
    qk.free_all()
    d, eff, E, k = 2048, 768, 16, 4
    router, gate, up, down, h0 = o.synth_moe(91, d, eff, E, T)
    rh = qk.register_weight(router, E, d // 256, o.Q4_K)
    gh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in gate]
    uh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in up]
    dh = [qk.register_weight(w, d, eff // 256, o.Q6_K) for w in down]
    layer = device.MoELayer(rh, gh, uh, dh, k, d, eff)
    gain = o.to_fixed(np.abs(np.random.default_rng(3).standard_normal(d)) + 0.5, FA)
    gain_h = qk.register_i64(gain)
    xn = (h0 * 37).astype(np.int64)                               # an un-normalised residual stream
    hn = o.rmsnorm_fixed(xn, FA, 1, gain)
    ids_ref, gates_ref, moe_ref = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, hn, d, eff, FA, FW)
    x = torch.from_numpy(xn).cuda()
    out, ids, gates = layer.block(x, gain_h, FA, FW, 1)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref) and np.array_equal(gates.cpu().numpy(), gates_ref)
    assert np.array_equal(out.cpu().numpy(), xn + moe_ref)
    inplace = x.clone()
    layer.block(inplace, gain_h, FA, FW, 1, out=inplace)            # out may alias x
    assert np.array_equal(inplace.cpu().numpy(), xn + moe_ref)
    got = qk.moe_block(layer.handle, xn, k, FA, FW, gain_handle=gain_h)   # host-buffer entry of the same block
    assert got is not None and np.array_equal(got[0], xn + moe_ref) and np.array_equal(got[1], ids_ref)
    plain = qk.moe_block(layer.handle, hn, k, FA, FW)                    # no gain: moe(x) only
    assert plain is not None and np.array_equal(plain[0], moe_ref)
    qk.free_all()


@pytest.mark.parametrize("shift", [0, 20, 31])
def test_decode_block_norm_over_the_residual_magnitudes(qk, shift):
    """The one-token block normalises its row inside the first streaming kernel.  Small residuals take the loop whose range
    tests were settled once for the whole row; at 2^20 the mean square needs the 128-bit root; at 2^31 the row leaves the
    64-bit quotient and the element-wise path with the wide quotient and the bitwise root runs.  All equal the checker."""
    import torch

    from integer_inference_engine_b200 import device
    qk.free_all()
    d, eff, E, k = 2048, 768, 16, 4
    router, gate, up, down, h0 = o.synth_moe(93, d, eff, E, 1)
    rh = qk.register_weight(router, E, d // 256, o.Q4_K)
    gh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in gate]
    uh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in up]
    dh = [qk.register_weight(w, d, eff // 256, o.Q6_K) for w in down]
    layer = device.MoELayer(rh, gh, uh, dh, k, d, eff)
    gain = o.to_fixed(np.abs(np.random.default_rng(5).standard_normal(d)) + 0.5, FA)
    gain_h = qk.register_i64(gain)
    xn = (h0 * 37).astype(np.int64) << shift
    assert int(np.abs(xn).max()) < 1 << 57
    hn = o.rmsnorm_fixed(xn, FA, 1, gain)
    ids_ref, gates_ref, moe_ref = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, hn, d, eff, FA, FW)
    out, ids, gates = layer.block(torch.from_numpy(xn).cuda(), gain_h, FA, FW, 1)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref) and np.array_equal(gates.cpu().numpy(), gates_ref)
    assert np.array_equal(out.cpu().numpy(), xn + moe_ref)
    qk.free_all()


@pytest.mark.parametrize("d,eff,E,k,T", [(512, 256, 8, 2, 40), (2048, 768, 16, 4, 150), (256, 256, 4, 2, 300)])
def test_device_moe_prefill_tensor_core_path(qk, d, eff, E, k, T):
    """From a set token count on (lowered to 32 here) the block runs on the tcgen05 grouped GEMMs (router GEMM, dispatch, gate/up with
    fused SiLU, down with fused combine); outputs stay byte-identical to the CPU oracle.  Expert loads are
    uneven, some 128-pair slabs are partial, and one case has more than one slab per expert."""
    import torch

    from integer_inference_engine_b200 import device
    qk.free_all()
    layer, h, (ids_ref, gates_ref, out_ref) = _device_layer(qk, 7 + d + T, d, eff, E, k, T)
    qk.load_library().iie_set_tc_min_tokens(32)
    out, ids, gates = layer.forward(h, FA, FW)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert np.array_equal(gates.cpu().numpy(), gates_ref)
    assert np.array_equal(out.cpu().numpy(), out_ref)
    # the streamed kernels give the same bytes for the same call
    qk.load_library().iie_set_tc_min_tokens(1 << 40)
    out2, _, _ = layer.forward(h, FA, FW)
    qk.load_library().iie_set_tc_min_tokens(192)
    assert torch.equal(out, out2)
    qk.free_all()
