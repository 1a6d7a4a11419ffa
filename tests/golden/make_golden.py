"""Regenerate the golden vectors in this directory from the reference project's own Python code.

Run where the reference tree is mounted; its location must be given in IIE_REFERENCE_ROOT:

    IIE_REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py [fixture ...]

Without arguments every fixture is regenerated; with names (half_fixed, codec, linear, scalar, q1, moe,
attention, q1_decode, nmc_decode, engine_generate) only those.

Inputs come from the seeded generators in ``oracle/qk_oracle.py`` (so the fixtures only need to
store seeds and outputs); outputs come from the reference's modules ``nmc.qk_codec``,
``nmc.cohere2``, ``nmc._bonsai.fixedpoint`` and ``trinote.infer_int.reference_bonsai``.  The test
``tests/test_oracle_golden.py`` replays the same seeds through this repository's oracle and
compares bytes, which pins the oracle to the reference without the reference being present.
"""
from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
if "IIE_REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set IIE_REFERENCE_ROOT to the reference checkout")
REF = Path(os.environ["IIE_REFERENCE_ROOT"])
sys.path.insert(0, str(REF / "north-mini-code" / "src"))
sys.path.insert(0, str(REF / "bonsai" / "src"))
sys.path.insert(0, str(ROOT))

from nmc import cohere2 as c2                        # noqa: E402
from nmc import qk_codec as rq                       # noqa: E402
from nmc._bonsai import fixedpoint as rfp            # noqa: E402
from trinote.infer_int.reference_bonsai import q1_linear_ref   # noqa: E402

from oracle import qk_oracle as o                    # noqa: E402

FA, FW = 16, 24


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def ref_dequant(raw, out_f, nb, qtype, frac):
    fn = rq.dequant_q4k_tensor if qtype == 0 else rq.dequant_q6k_tensor
    return fn(raw, out_f * nb * 256, frac).reshape(out_f, nb * 256)


def half_fixture():
    bits = np.arange(65536, dtype=np.uint16)
    bits = bits[((bits >> 10) & 31) != 31]
    out = {}
    for frac in (24, 16, 11):
        v = np.array([int(round(float(h) * (1 << frac))) for h in bits.view(np.float16)], dtype=np.int64)
        out[f"sha_{frac}"] = sha(v)
        out[f"sample_{frac}"] = v[::251]
    return out


def codec_fixture():
    out = {}
    for seed in (0, 1):
        rng = np.random.default_rng(100 + seed)
        r4, r6 = o.synth_q4k(rng, 3, 2), o.synth_q6k(rng, 3, 2)
        out[f"q4k_{seed}"] = ref_dequant(r4, 3, 2, 0, FW)
        out[f"q6k_{seed}"] = ref_dequant(r6, 3, 2, 1, FW)
        out[f"q4k_f16_{seed}"] = ref_dequant(r4, 3, 2, 0, 16)
    # the reference's own block generators, scalar decoder
    b4, b6 = rq.random_q4k(7), rq.random_q6k(7)
    out["ref_q4k_raw"] = np.frombuffer(np.float16(b4["d"]).tobytes() + np.float16(b4["dmin"]).tobytes()
                                       + b4["scales"].tobytes() + b4["qs"].tobytes(), np.uint8)
    out["ref_q4k_int"] = rq.dequant_q4k_int(**b4, frac=FW)
    out["ref_q6k_raw"] = np.frombuffer(b6["ql"].tobytes() + b6["qh"].tobytes() + b6["scales"].tobytes()
                                       + np.float16(b6["d"]).tobytes(), np.uint8)
    out["ref_q6k_int"] = rq.dequant_q6k_int(**b6, frac=FW)
    return out


def linear_fixture():
    out = {}
    for i, (qt, out_f, nb, T, magbits) in enumerate(LINEAR_CASES):
        rng = np.random.default_rng(200 + i)
        raw = (o.synth_q4k if qt == 0 else o.synth_q6k)(rng, out_f, nb)
        x = rng.integers(-(1 << magbits), 1 << magbits, size=(T, nb * 256), dtype=np.int64)
        out[f"y_{i}"] = c2.linear(x, ref_dequant(raw, out_f, nb, qt, FW), FW)
    return out


def scalar_fixture():
    rng = np.random.default_rng(300)
    x = np.concatenate([rng.integers(-(1 << 22), 1 << 22, size=4000), rng.integers(-(1 << 40), 1 << 40, size=500),
                        np.array([0, 1, -1, 65536, -65536, (1 << 62), -(1 << 62), np.iinfo(np.int64).max,
                                  np.iinfo(np.int64).min, 851968, -851968, 851967])]).astype(np.int64)
    safe = x[np.abs(x.astype(object)) < (1 << 46)].astype(np.int64)
    xx = rng.integers(-(1 << 18), 1 << 18, size=(3, 256), dtype=np.int64)
    g = rng.integers(1 << 15, 1 << 17, size=256, dtype=np.int64)
    lg = rng.integers(-4, 4, size=(12, 16), dtype=np.int64)
    return {"x": x, "sigmoid": rfp.fixed_point_sigmoid(x, FA), "sigmoid_f20": rfp.fixed_point_sigmoid(x, 20),
            "silu_x": safe, "silu": c2.silu_int(safe, FA),
            "rms_x": xx, "rms_g": g, "rms": rfp.fixed_point_rmsnorm(xx, FA, 1, gain_q=g),
            "topk_logits": lg, "topk": np.stack([c2._topk_lowidx(r, 5) for r in lg])}


class _LazyExperts:
    """Dequantise an expert's matrix with the reference codec only when the router selects it."""
    def __init__(self, raws, out_f, nb, qt): self.raws, self.out_f, self.nb, self.qt = raws, out_f, nb, qt
    def __getitem__(self, e): return ref_dequant(self.raws[e], self.out_f, self.nb, self.qt, FW)


synth_moe = o.synth_moe
LINEAR_CASES = o.GOLDEN_LINEAR_CASES


MOE_CASES = o.GOLDEN_MOE_CASES


def moe_fixture():
    out = {}
    for name, (seed, d, eff, E, k, T) in MOE_CASES.items():
        router, gate, up, down, h = synth_moe(seed, d, eff, E, T)
        cfg = c2.Cfg(d_model=d, n_heads=1, n_kv=1, head_dim=d, ffn=eff, vocab=1, n_experts=E, n_used=k,
                     expert_ffn=eff, fa=FA, fw=FW)
        We = {"router": ref_dequant(router, E, d // 256, 0, FW), "gate": _LazyExperts(gate, eff, d // 256, 0),
              "up": _LazyExperts(up, eff, d // 256, 0), "down": _LazyExperts(down, d, eff // 256, 1)}
        logits = c2.linear(h, We["router"], FW)
        out[f"{name}_ids"] = np.stack([c2._topk_lowidx(r, k) for r in logits]).astype(np.int32)
        out[f"{name}_out"] = c2.moe_layer_int(h, We, cfg)
        print(name, "done", flush=True)
    return out


def q1_fixture():
    out = {}
    for i, (out_f, nb, T, magbits) in enumerate([(7, 3, 1, 20), (7, 3, 3, 20), (16, 2, 2, 62)]):
        rng = np.random.default_rng(500 + i)
        bits, scale = o.synth_q1(rng, out_f, nb)
        if magbits > 40:
            scale = rng.integers(-(1 << 40), 1 << 40, size=scale.shape, dtype=np.int64)
        x = rng.integers(-(1 << magbits), 1 << magbits, size=(T, nb * 128), dtype=np.int64)
        out[f"y_{i}"] = q1_linear_ref(x, bits, scale, 16)
    return out


def attention_fixture():
    """RoPE (both pairings), softmax rows incl. masked sentinels, and KV-cached attention (decode and a short
    prefill, full and sliding-window) from the reference's own functions."""
    from nmc._bonsai import rope as rrope
    from nmc._bonsai import rope_v2 as rrope2
    out = {}
    rng = np.random.default_rng(700)
    cos, sin = rrope.build_rope_tables(40, 16, 50000.0, FA)
    out["rope_cos"], out["rope_sin"] = cos, sin
    x = rng.integers(-(1 << 22), 1 << 22, size=(3, 40, 16), dtype=np.int64)
    out["rope_inter"] = rrope.apply_rope_fixed(x, cos, sin, FA)
    out["rope_neox"] = rrope2.apply_rope_fixed_neox(x, cos, sin, FA)
    z = rng.integers(-(1 << 20), 1 << 20, size=(6, 50), dtype=np.int64)
    z[1, 10:] = -(1 << (FA + 30)); z[2, :] = 7; z[3, 0] = 1 << 40
    out["softmax"] = rfp.fixed_point_softmax(z, FA)
    H, Hkv, hd = 4, 2, 16
    cfg = c2.Cfg(d_model=H * hd, n_heads=H, n_kv=Hkv, head_dim=hd, ffn=0, vocab=0)
    for name, (Lc, m, window) in {"dec_full": (37, 1, None), "dec_win": (37, 1, 9), "pre_full": (12, 12, None),
                                  "pre_win": (20, 5, 7)}.items():
        r2 = np.random.default_rng(710 + len(name) + Lc)
        q = r2.integers(-(1 << 19), 1 << 19, size=(m, H, hd), dtype=np.int64)
        ck = r2.integers(-(1 << 19), 1 << 19, size=(Hkv, Lc, hd), dtype=np.int64)
        cv = r2.integers(-(1 << 19), 1 << 19, size=(Hkv, Lc, hd), dtype=np.int64)
        out[f"att_{name}"] = c2.attention_cached(q, ck, cv, Lc - m, cfg, window)
    return out


def q1_decode_fixture():
    """One KV-cached decode token of the reference's 1-bit decoder (reference_bonsai.py _run_layers) on a small
    random artifact with non-trivial gains and scales: a 5-token prefill through the reference fills the cache, the
    sixth token is the recorded step."""
    from trinote.infer_int import reference_bonsai as rb
    cfgp = {"dModel": 256, "nHeads": 4, "nHeadsKv": 2, "headDim": 64, "dFfn": 256, "vocab": 96, "nLayers": 2,
            "fpFracBits": 16, "ropeBase": 10000}
    art = rb.random_bonsai_artifact(cfgp, seq_len=8, seed=77)
    rng = np.random.default_rng(78)
    for layer in art["layers"] + [art]:
        for key in list(layer):
            if key.endswith("_gain_fp"):
                layer[key] = np.rint((np.abs(rng.standard_normal(layer[key].shape)) + 0.5) * 65536).astype(np.int64)
            if key.endswith("_scale_fp"):
                sc = np.abs(rng.standard_normal(layer[key].shape) * 0.03).astype(np.float16)
                layer[key] = np.rint(sc.astype(np.float64) * 65536).astype(np.int64)
    model = rb.BonsaiReferenceModel(artifact=art)
    cache = rb._BonsaiKVCache(2)
    prompt = [3, 90, 41, 7, 66]
    x_prompt = model._run_layers(prompt, cache)
    out = {"cos": art["cos_fp"], "sin": art["sin_fp"], "token": np.int64(12), "pos": np.int64(5)}
    # the prefill itself: embedded prompt rows, the last position's logits (what forward(..., last_only=True) returns;
    # the K/V rows it leaves are k0/v0, k1/v1 below)
    out["prompt"] = np.asarray(prompt, dtype=np.int64)
    out["prompt_embed"] = rb.q1_rows_fp(art["embed_bits"], art["embed_scale_fp"], out["prompt"], 16)
    out["prefill_logits"] = model._output_linear(rb._rmsnorm(x_prompt[-1:], 16, art["final_norm_gain_fp"]), 16, fast=False)
    for li in range(2):
        out[f"k{li}"], out[f"v{li}"] = cache.k[li].copy(), cache.v[li].copy()
    x = model._run_layers([12], cache)
    frac = 16
    xn = rb._rmsnorm(x, frac, art["final_norm_gain_fp"])
    logits = model._output_linear(xn, frac, fast=False)
    out["x"], out["logits"], out["next"] = x, logits, np.int64(int(logits.argmax(axis=1)[0]))
    for li in range(2):
        out[f"k{li}_after"], out[f"v{li}_after"] = cache.k[li].copy(), cache.v[li].copy()
        for key, val in art["layers"][li].items():
            out[f"L{li}_{key}"] = val
    for key in ("embed_bits", "embed_scale_fp", "output_bits", "output_scale_fp", "final_norm_gain_fp"):
        out[key] = art[key]
    return out


def nmc_decode_fixture():
    """KV-cached decode steps of the reference's own parallel MoE block and tied head (cohere2.py block_cached,
    tied_head_int, generate) on the small synthetic decoder ``oracle.qk_oracle.synth_decoder`` describes: layer 0
    attends to everything without rotation, layer 1 through a sliding window with interleaved RoPE.  A prompt of
    ``NMC_DECODE_CASE['prompt']`` tokens fills the cache through the reference; the recorded values are the cache
    before and after, the row after every block, the logits and the greedy picks of the next decode steps."""
    case = o.NMC_DECODE_CASE
    m = o.synth_decoder(case["seed"], case)
    d, H, Hkv, hd, eff, E, k, vocab = (case[n] for n in ("d", "H", "Hkv", "hd", "eff", "E", "k", "vocab"))
    nb = d // 256
    cfg = c2.Cfg(d_model=d, n_heads=H, n_kv=Hkv, head_dim=hd, ffn=eff, vocab=vocab, n_experts=E, n_used=k,
                 expert_ffn=eff, sliding_window=case["window"], rope_base=case["rope_base"], fa=FA, fw=FW)
    from nmc._bonsai import rope as rrope
    cos, sin = rrope.build_rope_tables(case["rows"], hd, case["rope_base"], FA)
    layers = []
    for L in m["layers"]:
        W = {"attn_norm": L["gain"], "wq": ref_dequant(L["wq"], H * hd, nb, 0, FW), "wk": ref_dequant(L["wk"], Hkv * hd, nb, 0, FW),
             "wv": ref_dequant(L["wv"], Hkv * hd, nb, 0, FW), "wo": ref_dequant(L["wo"], d, H * hd // 256, 0, FW)}
        router, gate, up, down = L["moe"]
        We = {"router": ref_dequant(router, E, nb, 0, FW), "gate": _LazyExperts(gate, eff, nb, 0),
              "up": _LazyExperts(up, eff, nb, 0), "down": _LazyExperts(down, d, eff // 256, 1)}
        layers.append((W, We))
    table = ref_dequant(m["embd"], vocab, nb, 1, FA)
    head_W = {"output_norm": m["out_gain"], "token_embd": ref_dequant(m["embd"], vocab, nb, 1, FW)}
    embed = lambda t: table[t]
    cache = c2.KVCache(len(layers), max_length=case["rows"])
    prompt = list(case["prompt"])
    last = c2._run_layers_cached(np.stack([embed(t) for t in prompt]), layers, cfg, cos, sin, cache)[-1:]
    out = {"cos": cos, "sin": sin}
    for li in range(len(layers)):
        out[f"k{li}"], out[f"v{li}"] = cache.k[li].copy(), cache.v[li].copy()
    tok = int(np.argmax(c2.tied_head_int(last, head_W, cfg)[0]))          # first pick: after the prompt
    picks, xs, logit_rows = [tok], [], []
    for step in range(case["steps"]):
        x = embed(tok)[None, :]
        rows = [x.copy()]
        for li, (W, We) in enumerate(layers):
            x = c2.block_cached(x, W, We, cfg, cos, sin, cache, li, c2.window_for_layer(cfg, li))
            rows.append(x.copy())
        logits = c2.tied_head_int(x, head_W, cfg)[0]
        tok = int(np.flatnonzero(logits == logits.max())[0])
        picks.append(tok); xs.append(np.concatenate(rows)); logit_rows.append(logits)
    out["picks"], out["x"], out["logits"] = np.array(picks, np.int64), np.stack(xs), np.stack(logit_rows)
    for li in range(len(layers)):
        out[f"k{li}_after"], out[f"v{li}_after"] = cache.k[li].copy(), cache.v[li].copy()
    # the library's own generate() on the same inputs yields the same picks (its pick receives the logits row)
    gen = c2.generate(prompt, embed, layers, head_W, cfg, cos, sin, case["steps"] + 1,
                      lambda lg, pos, hist: int(np.flatnonzero(lg == lg.max())[0]))
    assert gen == picks, (gen, picks)
    return out


def engine_generate_fixture():
    """Greedy generation by the reference's own ``Engine`` (engine.py:535-597) on its CPU backend, for the synthetic GGUF
    checkpoint ``integer_inference_engine_b200.gguf.write_synthetic_model`` writes with ``oracle.qk_oracle.ENGINE_CASE``;
    the CPU kernel it binds is the one ``oracle/build.py`` compiles from the reference (BONSAI_BIN_DIR)."""
    import tempfile
    from integer_inference_engine_b200 import gguf as ours
    case = o.ENGINE_CASE
    os.environ["BONSAI_BIN_DIR"] = str(ROOT / "oracle" / "_ref")
    from nmc.engine import Engine
    with tempfile.TemporaryDirectory() as tmp:
        shape = ours.write_synthetic_model(Path(tmp) / "m.gguf", **case["model"])
        ours.write_stub_tokenizer(Path(tmp) / "tok", shape["vocab"])
        eng = Engine(str(Path(tmp) / "m.gguf"), str(Path(tmp) / "tok"), backend="cpu")
        ids = eng.generate(list(case["prompt"]), case["n_new"], stop_eos=False)
    return {"ids": np.array(ids, np.int64)}


FIXTURES = {"engine_generate": engine_generate_fixture, "half_fixed": half_fixture, "codec": codec_fixture, "linear": linear_fixture, "scalar": scalar_fixture,
            "q1": q1_fixture, "moe": moe_fixture, "attention": attention_fixture, "q1_decode": q1_decode_fixture,
            "nmc_decode": nmc_decode_fixture}


def main():
    for name in (sys.argv[1:] or list(FIXTURES)):
        np.savez_compressed(HERE / f"{name}.npz", **FIXTURES[name]())
        print("wrote", name, flush=True)


if __name__ == "__main__":
    main()
