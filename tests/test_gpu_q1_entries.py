"""GPU parity of the 1-bit decoder's whole-model entries under the reference's names (bonsai_buf_upload_i64,
bonsai_prefill_forward_gpu, bonsai_decode_ctx_*, bonsai_decode_step, bonsai_attention_prefill_gpu,
bonsai_attention_decode_batched_gpu), through the bridge functions named as in
bonsai/src/trinote/infer_int/gpu_native.py:418-595.

Expected values are the reference's own: ``tests/golden/q1_decode.npz`` holds a 5-token prefill (the K/V rows it leaves,
its last-position logits) and the decode step after it, recorded from ``BonsaiReferenceModel`` on its host path."""
import numpy as np
import pytest

from oracle import model_oracle
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FRAC = 16


@pytest.fixture(scope="module")
def model(golden_dir):
    from integer_inference_engine_b200 import q1_gpu
    assert q1_gpu.monolith_available(), "the CUDA library must be built and a GPU present"
    g = np.load(golden_dir / "q1_decode.npz")
    reg = lambda prefix: q1_gpu.q1_register_weight(g[f"{prefix}_bits"], g[f"{prefix}_scale_fp"])
    w = {name: [reg(f"L{li}_{name}") for li in range(2)] for name in ("wq", "wk", "wv", "wo", "w1", "wu", "w2")}
    gains = {"n1g": "n1_gain_fp", "n2g": "n2_gain_fp", "qng": "q_norm_gain_fp", "kng": "k_norm_gain_fp"}
    gh = {name: [q1_gpu.buf_upload_i64(g[f"L{li}_{key}"]) for li in range(2)] for name, key in gains.items()}
    w["out_head"], w["out_head_vocab"] = reg("output"), 96
    gh["finalg"], gh["cos_h"], gh["sin_h"] = (q1_gpu.buf_upload_i64(g[k]) for k in ("final_norm_gain_fp", "cos", "sin"))
    assert None not in gh.values() and all(None not in v for v in gh.values() if isinstance(v, list))
    dims = dict(d=256, H=4, Hkv=2, hd=64, dff=256, vocab=96, layers=2)
    inv_sqrt = round((1.0 / np.sqrt(64)) * (1 << FRAC))
    yield g, w, gh, dims, inv_sqrt
    q1_gpu.q1_free_weights()


def test_prefill_forward_matches_the_reference_prefill(model):
    from integer_inference_engine_b200 import q1_gpu
    g, w, gh, s, inv_sqrt = model
    T = int(g["prompt"].size)
    dims = (T, s["d"], s["layers"], s["H"], s["Hkv"], s["hd"], s["dff"])
    logits, k, v = q1_gpu.prefill_forward_gpu(g["prompt_embed"], dims, w, gh, FRAC, 1, inv_sqrt, export_kv=True)
    assert np.array_equal(logits, g["prefill_logits"][0])
    for li in range(2):
        assert np.array_equal(k[li], g[f"k{li}"]) and np.array_equal(v[li], g[f"v{li}"]), li
    only = q1_gpu.prefill_forward_gpu(g["prompt_embed"], dims, w, gh, FRAC, 1, inv_sqrt)
    assert np.array_equal(only, logits)
    # one token is a prefill too
    one = q1_gpu.prefill_forward_gpu(g["prompt_embed"][:1], (1,) + dims[1:], w, gh, FRAC, 1, inv_sqrt, export_kv=True)
    assert np.array_equal(one[1][0], g["k0"][:, :1]) and np.array_equal(one[2][1], g["v1"][:, :1])
    # an activation outside the norm's envelope: the overflow answer, not wrong bytes
    bad = g["prompt_embed"].copy()
    bad[2, :2] = np.iinfo(np.int64).min
    assert q1_gpu.prefill_forward_gpu(bad, dims, w, gh, FRAC, 1, inv_sqrt) is None
    # handle lists of the wrong length and handles of the wrong kind are refused
    with pytest.raises(ValueError):
        q1_gpu.prefill_forward_gpu(g["prompt_embed"], dims, {**w, "wq": w["wq"][:1]}, gh, FRAC, 1, inv_sqrt)
    assert q1_gpu.prefill_forward_gpu(g["prompt_embed"], dims, {**w, "wq": w["wk"]}, gh, FRAC, 1, inv_sqrt) is None


def test_decode_context_steps_sequences_at_their_own_positions(model):
    from integer_inference_engine_b200 import q1_gpu
    g, w, gh, s, inv_sqrt = model
    cap = 8
    dims = (2, s["layers"], s["H"], s["Hkv"], s["hd"], s["d"], s["dff"], s["vocab"])
    ctx = q1_gpu.decode_ctx_create(dims, w, gh, FRAC, 1, inv_sqrt, cap)
    assert ctx is not None
    full_k = np.stack([g["k0"], g["k1"]]); full_v = np.stack([g["v0"], g["v1"]])
    # sequence 0: the whole recorded prefill, then the recorded step (token 12 at position 5)
    # sequence 1: the first three prompt tokens, then the fourth prompt token at position 3
    assert q1_gpu.decode_ctx_seed_seq(ctx, 0, full_k, full_v)
    assert q1_gpu.decode_ctx_seed_seq(ctx, 1, full_k[:, :, :3], full_v[:, :, :3])
    x0 = model_oracle.q1_rows(g["embed_bits"], g["embed_scale_fp"], int(g["token"]))
    x = np.concatenate([x0, g["prompt_embed"][3:4]])
    logits = q1_gpu.decode_step(ctx, x, [5, 3], s["vocab"])
    assert logits is not None
    assert np.array_equal(logits[0], g["logits"][0]) and int(logits[0].argmax()) == int(g["next"])
    # sequence 1 has now seen prompt[:4]: a prefill of those four tokens gives the same last-position logits
    T4 = (4, s["d"], s["layers"], s["H"], s["Hkv"], s["hd"], s["dff"])
    want = q1_gpu.prefill_forward_gpu(g["prompt_embed"][:4], T4, w, gh, FRAC, 1, inv_sqrt)
    assert np.array_equal(logits[1], want)
    # next step of sequence 1 (fifth prompt token at position 4) must land on the recorded prefill logits
    again = q1_gpu.decode_step(ctx, np.concatenate([x0, g["prompt_embed"][4:5]]), [6, 4], s["vocab"])
    assert np.array_equal(again[1], g["prefill_logits"][0])
    assert q1_gpu.decode_step(ctx, x, [5, cap], s["vocab"]) is None          # a position beyond the cache
    q1_gpu.decode_ctx_free(ctx)
    q1_gpu.decode_ctx_free(ctx)                                               # freeing twice is harmless
    assert q1_gpu.decode_step(ctx, x, [5, 3], s["vocab"]) is None


def _host_attention(q, k, v, start, frac, inv_sqrt):
    """q (H, M, hd), k / v (Hkv, L, hd) -> (H, M, hd) with the checker's cached attention (token-major layout)."""
    H, M, hd = q.shape
    out = o.attention_cached(np.transpose(q, (1, 0, 2)), k, v, start, H, k.shape[0], frac, None, inv_sqrt)
    return np.transpose(out.reshape(M, H, hd), (1, 0, 2))


@pytest.mark.parametrize(("H", "Hkv", "hd", "M", "start"), ((4, 2, 64, 5, 0), (8, 2, 64, 3, 4), (4, 4, 128, 1, 6), (4, 4, 16, 8, 0), (2, 1, 8, 4, 2)))
def test_standalone_prefill_attention(H, Hkv, hd, M, start):
    from integer_inference_engine_b200 import q1_gpu
    rng = np.random.default_rng(H * 100 + M)
    L = start + M
    q = rng.integers(-(1 << 17), 1 << 17, size=(H, M, hd), dtype=np.int64)
    k = rng.integers(-(1 << 17), 1 << 17, size=(Hkv, L, hd), dtype=np.int64)
    v = rng.integers(-(1 << 17), 1 << 17, size=(Hkv, L, hd), dtype=np.int64)
    inv_sqrt = round((1.0 / np.sqrt(hd)) * (1 << FRAC))
    got = q1_gpu.attention_prefill_gpu(q, k, v, start, FRAC, inv_sqrt)
    assert np.array_equal(got, _host_attention(q, k, v, start, FRAC, inv_sqrt))
    wide = v.copy()
    wide[0, 0, 0] = 1 << 40
    assert q1_gpu.attention_prefill_gpu(q, k, wide, start, FRAC, inv_sqrt) is None     # beyond the int32 rows: host path
    with pytest.raises(ValueError):
        q1_gpu.attention_prefill_gpu(q, k[:, :-1], v[:, :-1], start, FRAC, inv_sqrt)


def test_standalone_batched_decode_attention():
    from integer_inference_engine_b200 import q1_gpu
    rng = np.random.default_rng(9)
    B, H, Hkv, hd, cap = 3, 4, 2, 64, 7
    q = rng.integers(-(1 << 17), 1 << 17, size=(B, H, hd), dtype=np.int64)
    K = rng.integers(-(1 << 17), 1 << 17, size=(B, Hkv, cap, hd), dtype=np.int64)
    V = rng.integers(-(1 << 17), 1 << 17, size=(B, Hkv, cap, hd), dtype=np.int64)
    lengths = np.array([7, 1, 4], dtype=np.int64)
    K[1, :, 3:] = 1 << 50                                     # padding beyond a sequence's length is never read as a value
    inv_sqrt = round((1.0 / np.sqrt(hd)) * (1 << FRAC))
    got = q1_gpu.attention_decode_batched_gpu(q, K, V, lengths, FRAC, inv_sqrt)
    assert got is not None
    for b in range(B):
        n = int(lengths[b])
        want = _host_attention(q[b][:, None, :], K[b][:, :n], V[b][:, :n], n - 1, FRAC, inv_sqrt)
        assert np.array_equal(got[b], want[:, 0, :]), b
    assert q1_gpu.attention_decode_batched_gpu(q, K, V, np.array([7, 4, 4]), FRAC, inv_sqrt) is None   # now the wide rows count
