"""CPU suite: the NumPy and C oracles reproduce the committed golden vectors, which were produced by
the reference project's own Python code (tests/golden/make_golden.py)."""
import hashlib

import numpy as np
import pytest

from oracle import native as onat
from oracle import qk_oracle as o

FA, FW = 16, 24


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _finite_halves():
    bits = np.arange(65536, dtype=np.uint16)
    return bits[((bits >> 10) & 31) != 31]


@pytest.mark.parametrize("frac", [24, 16, 11])
def test_half_to_fixed_all_finite_halves(golden_dir, frac):
    g = np.load(golden_dir / "half_fixed.npz")
    bits = _finite_halves()
    v = o.half_bits_to_fixed(bits, frac)
    assert _sha(v) == str(g[f"sha_{frac}"])
    assert np.array_equal(v[::251], g[f"sample_{frac}"])
    lib = onat.orc()
    c = np.array([lib.orc_half_to_fixed(int(b), frac) for b in bits[::7]], dtype=np.int64)
    assert np.array_equal(c, v[::7])


def test_half_at_weight_scale_is_a_pure_shift():
    """At frac 24 every finite half times 2**24 is an integer, so no rounding ever fires."""
    bits = _finite_halves()
    exact = np.array([int(float(h) * (1 << 24)) for h in bits.view(np.float16)], dtype=np.int64)
    assert np.array_equal(o.half_bits_to_fixed(bits, 24), exact)


def test_block_codecs(golden_dir):
    g = np.load(golden_dir / "codec.npz")
    for seed in (0, 1):
        rng = np.random.default_rng(100 + seed)
        r4, r6 = o.synth_q4k(rng, 3, 2), o.synth_q6k(rng, 3, 2)
        assert np.array_equal(o.dequant(r4, 3, 2, o.Q4_K, FW), g[f"q4k_{seed}"])
        assert np.array_equal(o.dequant(r6, 3, 2, o.Q6_K, FW), g[f"q6k_{seed}"])
        assert np.array_equal(o.dequant(r4, 3, 2, o.Q4_K, 16), g[f"q4k_f16_{seed}"])
    assert np.array_equal(o.dequant_q4k(g["ref_q4k_raw"].tobytes(), 1, FW), g["ref_q4k_int"])
    assert np.array_equal(o.dequant_q6k(g["ref_q6k_raw"].tobytes(), 1, FW), g["ref_q6k_int"])


def _linear_case(i):
    qt, out_f, nb, T, magbits = o.GOLDEN_LINEAR_CASES[i]
    rng = np.random.default_rng(200 + i)
    raw = (o.synth_q4k if qt == 0 else o.synth_q6k)(rng, out_f, nb)
    x = rng.integers(-(1 << magbits), 1 << magbits, size=(T, nb * 256), dtype=np.int64)
    return qt, out_f, nb, raw, x


@pytest.mark.parametrize("i", range(len(o.GOLDEN_LINEAR_CASES)))
def test_fused_linear(golden_dir, i):
    g = np.load(golden_dir / "linear.npz")
    qt, out_f, nb, raw, x = _linear_case(i)
    assert np.array_equal(o.qk_linear(raw, x, out_f, nb, FW, qt), g[f"y_{i}"])
    assert np.array_equal(onat.qk_linear(raw, x, out_f, nb, FW, qt), g[f"y_{i}"])
    if onat.ref_available():
        assert np.array_equal(onat.ref_qk_linear(raw, x, out_f, nb, FW, qt), g[f"y_{i}"])


def test_scalar_functions(golden_dir):
    g = np.load(golden_dir / "scalar.npz")
    assert np.array_equal(o.sigmoid_fixed(g["x"], FA), g["sigmoid"])
    assert np.array_equal(o.sigmoid_fixed(g["x"], 20), g["sigmoid_f20"])
    assert np.array_equal(onat.sigmoid(g["x"], FA), g["sigmoid"])
    assert np.array_equal(onat.sigmoid(g["x"], 20), g["sigmoid_f20"])
    assert np.array_equal(o.silu_int(g["silu_x"], FA), g["silu"])
    assert np.array_equal(onat.silu(g["silu_x"], FA), g["silu"])
    assert np.array_equal(o.rmsnorm_fixed(g["rms_x"], FA, 1, g["rms_g"]), g["rms"])
    for row, want in zip(g["topk_logits"], g["topk"]):
        assert np.array_equal(o.topk_lowidx(row, 5), want)
        assert np.array_equal(onat.topk_lowidx(row, 5), want)


def test_topk_all_equal_keeps_ascending_ids():
    assert o.topk_lowidx(np.zeros(16, np.int64), 4).tolist() == [0, 1, 2, 3]
    assert onat.topk_lowidx(np.zeros(16, np.int64), 4).tolist() == [0, 1, 2, 3]


@pytest.mark.parametrize("name", ["small", "config1"])
def test_moe_block(golden_dir, name):
    """The whole MoE FFN (router ids and block output) against the reference's moe_layer_int."""
    g = np.load(golden_dir / "moe.npz")
    seed, d, eff, E, k, T = o.GOLDEN_MOE_CASES[name]
    router, gate, up, down, h = o.synth_moe(seed, d, eff, E, T)
    ids, gates, out = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, h, d, eff, FA, FW)
    assert np.array_equal(ids, g[f"{name}_ids"])
    assert np.array_equal(out, g[f"{name}_out"])
    if name == "small":                      # the pure NumPy restatement as well (slow at full size)
        def experts(e):
            return (o.dequant(gate[e], eff, d // 256, o.Q4_K, FW), o.dequant(up[e], eff, d // 256, o.Q4_K, FW),
                    o.dequant(down[e], d, eff // 256, o.Q6_K, FW))
        ids2, gates2, out2 = o.moe_layer(h, o.dequant(router, E, d // 256, o.Q4_K, FW), experts, k, FA, FW)
        assert np.array_equal(ids2, ids) and np.array_equal(gates2, gates) and np.array_equal(out2, out)


def test_q1_linear(golden_dir):
    g = np.load(golden_dir / "q1.npz")
    for i, (out_f, nb, T, magbits) in enumerate([(7, 3, 1, 20), (7, 3, 3, 20), (16, 2, 2, 62)]):
        rng = np.random.default_rng(500 + i)
        bits, scale = o.synth_q1(rng, out_f, nb)
        if magbits > 40:
            scale = rng.integers(-(1 << 40), 1 << 40, size=scale.shape, dtype=np.int64)
        x = rng.integers(-(1 << magbits), 1 << magbits, size=(T, nb * 128), dtype=np.int64)
        assert np.array_equal(o.q1_linear(x, bits, scale, 16), g[f"y_{i}"])
        assert np.array_equal(onat.q1_linear(x, bits, scale, 16), g[f"y_{i}"])


def test_balanced_limbs_capacity_and_roundtrip():
    """Digit-count rule: exact up to 127*(256^L-1)/255, e.g. two digits fail on 32640..32767."""
    assert o.balanced_capacity(2) == 32639
    assert o.limbs_needed(32639) == 2 and o.limbs_needed(32640) == 3
    rng = np.random.default_rng(9)
    x = rng.integers(-(1 << 62), 1 << 62, size=2000, dtype=np.int64)
    d = o.balanced_limbs(x, 8).astype(object)
    back = sum(d[l] * (256 ** l) for l in range(8))
    assert np.array_equal(np.asarray(back, dtype=object), x.astype(object))
    with pytest.raises(OverflowError):
        o.limbs_needed(o.balanced_capacity(8) + 1)


def test_attention_rope_softmax(golden_dir):
    """Same seeds as tests/golden/make_golden.py::attention_fixture; outputs are the reference's."""
    g = np.load(golden_dir / "attention.npz")
    rng = np.random.default_rng(700)
    cos, sin = o.build_rope_tables(40, 16, 50000.0, FA)
    assert np.array_equal(cos, g["rope_cos"]) and np.array_equal(sin, g["rope_sin"])
    x = rng.integers(-(1 << 22), 1 << 22, size=(3, 40, 16), dtype=np.int64)
    assert np.array_equal(o.rope_fixed(x, cos, sin, FA), g["rope_inter"])
    assert np.array_equal(o.rope_fixed(x, cos, sin, FA, neox=True), g["rope_neox"])
    z = rng.integers(-(1 << 20), 1 << 20, size=(6, 50), dtype=np.int64)
    z[1, 10:] = -(1 << (FA + 30)); z[2, :] = 7; z[3, 0] = 1 << 40
    assert np.array_equal(o.softmax_fixed(z, FA), g["softmax"])
    H, Hkv, hd = 4, 2, 16
    for name, (Lc, m, window) in {"dec_full": (37, 1, None), "dec_win": (37, 1, 9), "pre_full": (12, 12, None),
                                  "pre_win": (20, 5, 7)}.items():
        r2 = np.random.default_rng(710 + len(name) + Lc)
        q = r2.integers(-(1 << 19), 1 << 19, size=(m, H, hd), dtype=np.int64)
        ck = r2.integers(-(1 << 19), 1 << 19, size=(Hkv, Lc, hd), dtype=np.int64)
        cv = r2.integers(-(1 << 19), 1 << 19, size=(Hkv, Lc, hd), dtype=np.int64)
        assert np.array_equal(o.attention_cached(q, ck, cv, Lc - m, H, Hkv, FA, window), g[f"att_{name}"]), name


def q1_golden_layers(g, rows=None):
    """The 1-bit decode fixture (tests/golden/make_golden.py::q1_decode_fixture) in the checker's layer format."""
    layers = []
    for li in range(2):
        w = lambda n: (g[f"L{li}_{n}_bits"], g[f"L{li}_{n}_scale_fp"])
        cat = lambda *names: (np.concatenate([w(n)[0] for n in names]), np.concatenate([w(n)[1] for n in names]))
        k0, v0 = g[f"k{li}"], g[f"v{li}"]
        k = np.zeros((k0.shape[0], rows or k0.shape[1] + 1, k0.shape[2]), np.int64); k[:, :k0.shape[1]] = k0
        v = np.zeros_like(k); v[:, :v0.shape[1]] = v0
        layers.append({"n1": g[f"L{li}_n1_gain_fp"], "n2": g[f"L{li}_n2_gain_fp"], "qn": g[f"L{li}_q_norm_gain_fp"],
                       "kn": g[f"L{li}_k_norm_gain_fp"], "wqkv": cat("wq", "wk", "wv"), "wo": w("wo"), "w1u": cat("w1", "wu"),
                       "w2": w("w2"), "k": k, "v": v})
    top = {"embed": (g["embed_bits"], g["embed_scale_fp"]), "head": (g["output_bits"], g["output_scale_fp"]),
           "out_gain": g["final_norm_gain_fp"]}
    cfg = dict(d=256, H=4, Hkv=2, hd=64, ffn=256, frac=16)
    return layers, top, cfg


def test_q1_decode_token(golden_dir):
    """One KV-cached decode token of the reference's 1-bit decoder: hidden state, logits, pick and the appended
    cache rows are the reference's own."""
    from oracle import model_oracle
    g = np.load(golden_dir / "q1_decode.npz")
    layers, top, cfg = q1_golden_layers(g)
    pos = int(g["pos"])
    nxt, trace, logits = model_oracle.q1_decode_token(int(g["token"]), pos, layers, top, cfg, g["cos"], g["sin"])
    assert np.array_equal(trace[-1:], g["x"])
    assert np.array_equal(logits, g["logits"][0]) and nxt == int(g["next"])
    for li in range(2):
        assert np.array_equal(layers[li]["k"][:, :pos + 1], g[f"k{li}_after"])
        assert np.array_equal(layers[li]["v"][:, :pos + 1], g[f"v{li}_after"])


def nmc_golden_layers(g):
    """The decode-step fixture of the MoE decoder (tests/golden/make_golden.py::nmc_decode_fixture) in the checker's
    layer format: weights from the seeded generator, caches as the reference left them after the prompt."""
    case = o.NMC_DECODE_CASE
    m = o.synth_decoder(case["seed"], case)
    layers = []
    for li, L in enumerate(m["layers"]):
        k0, v0 = g[f"k{li}"], g[f"v{li}"]
        k = np.zeros((k0.shape[0], case["rows"], k0.shape[2]), np.int64); k[:, :k0.shape[1]] = k0
        v = np.zeros_like(k); v[:, :v0.shape[1]] = v0
        layers.append({"gain": L["gain"], "wq": L["wq"], "wk": L["wk"], "wv": L["wv"], "wo": L["wo"], "k": k, "v": v,
                       "full": li % 4 == 0, "moe": L["moe"]})
    cfg = dict(d=case["d"], H=case["H"], Hkv=case["Hkv"], hd=case["hd"], eff=case["eff"], E=case["E"], k=case["k"],
               vocab=case["vocab"], window=case["window"], fa=FA, fw=FW)
    return layers, m, cfg


def test_nmc_decode_steps(golden_dir):
    """Three KV-cached decode steps of the reference's parallel MoE block and tied head (cohere2.block_cached,
    tied_head_int): the row after every block, the logits, the greedy picks and the appended cache rows are the
    reference's own, for a full-attention block without rotation and a sliding-window block with RoPE."""
    from oracle import model_oracle
    g = np.load(golden_dir / "nmc_decode.npz")
    case = o.NMC_DECODE_CASE
    layers, m, cfg = nmc_golden_layers(g)
    cos, sin = o.build_rope_tables(case["rows"], case["hd"], case["rope_base"], FA)
    assert np.array_equal(cos, g["cos"]) and np.array_equal(sin, g["sin"])
    tok, pos = int(g["picks"][0]), len(case["prompt"])
    for step in range(case["steps"]):
        tok, trace, logits = model_oracle.decode_token(tok, pos + step, layers, m["embd"], m["out_gain"], cfg, cos, sin)
        assert np.array_equal(trace, g["x"][step]), step
        assert np.array_equal(logits, g["logits"][step]) and tok == int(g["picks"][step + 1])
    for li in range(case["layers"]):
        n = pos + case["steps"]
        assert np.array_equal(layers[li]["k"][:, :n], g[f"k{li}_after"]) and np.array_equal(layers[li]["v"][:, :n], g[f"v{li}_after"])
