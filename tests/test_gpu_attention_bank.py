"""GPU parity of the request-scoped attention bank through the reference's own entry names
(qk_attention_bank_create / import / apply / reset / destroy and the bridge class over them): device
Q/K/V -> RoPE -> K/V append -> exact attention -> O equals the host composition byte for byte."""
import numpy as np
import pytest

from integer_inference_engine_b200 import qk_cuda
from oracle import native as onat
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FA, FW = 16, 24


@pytest.mark.parametrize(("d_model", "heads", "n_kv", "head_dim"), ((256, 8, 2, 64), (512, 4, 2, 64), (512, 8, 1, 128)),
                         ids=("query-wider-than-hidden", "hidden-wider-than-query", "one-kv-head"))
def test_resident_attention_decode_matches_host_cache(d_model, heads, n_kv, head_dim):
    assert qk_cuda.resident_attention_available()
    qk_cuda.free_all()
    rng = np.random.default_rng(1701)
    max_length = 8
    nb, q_width = d_model // 256, heads * head_dim
    q_nb = q_width // 256

    def make_weight(out_f, qtype, seed, in_blocks=nb):
        raw = (o.synth_q4k if qtype == o.Q4_K else o.synth_q6k)(np.random.default_rng(seed), out_f, in_blocks)
        return raw, qk_cuda.register_weight(raw, out_f, in_blocks, qtype)

    qraw, qh = make_weight(q_width, o.Q4_K, 20000)
    kraw, kh = make_weight(n_kv * head_dim, o.Q6_K, 21000)
    vraw, vh = make_weight(n_kv * head_dim, o.Q4_K, 22000)
    oraw, oh = make_weight(d_model, o.Q6_K, 23000, q_nb)
    cos, sin = o.build_rope_tables(max_length, head_dim, 50000.0, FA)
    bank = qk_cuda.ResidentAttentionCache(1, max_length, d_model, heads, n_kv, head_dim, FA, cos, sin)
    start = 3
    ck = rng.integers(-(1 << 17), 1 << 17, size=(n_kv, start, head_dim), dtype=np.int64)
    cv = rng.integers(-(1 << 17), 1 << 17, size=(n_kv, start, head_dim), dtype=np.int64)
    bank.import_layer(0, ck, cv)
    assert bank.workspace_bytes() >= 2 * n_kv * max_length * head_dim * 4

    # declarations with the wrong widths are refused before any K/V row is written
    _, wrong_qh = make_weight(q_width + 16, o.Q4_K, 24000)
    _, wrong_oh = make_weight(d_model, o.Q6_K, 25000, q_nb + 1)
    _, wrong_kh = make_weight(n_kv * head_dim, o.Q6_K, 26000, nb + 1)
    probe = np.zeros((1, d_model), dtype=np.int64)
    with pytest.raises(ValueError, match="hidden row must be"):
        bank.apply(0, qh, kh, vh, oh, np.zeros((1, d_model + 1), dtype=np.int64), FW, None, False)
    for handles in ((wrong_qh, kh, vh, oh), (qh, wrong_kh, vh, oh), (qh, kh, wrong_kh, oh), (qh, kh, vh, wrong_oh)):
        with pytest.raises(qk_cuda.CudaContextError, match="native status"):
            bank.apply(0, *handles, probe, FW, None, False)
    assert bank.length(0) == start

    lin = lambda raw, qtype, x, out_f, in_blocks=nb: onat.qk_linear(raw, x, out_f, in_blocks, FW, qtype)
    for rope, window in ((True, 3), (False, None), (True, None), (False, 2)):
        x = rng.integers(-(1 << 17), 1 << 17, size=(1, d_model), dtype=np.int64)
        q = lin(qraw, o.Q4_K, x, q_width).reshape(1, heads, head_dim)
        k = lin(kraw, o.Q6_K, x, n_kv * head_dim).reshape(1, n_kv, head_dim)
        v = lin(vraw, o.Q4_K, x, n_kv * head_dim).reshape(1, n_kv, head_dim)
        if rope:
            rot = lambda t: o.rope_fixed(np.transpose(t, (1, 0, 2)), cos[start:start + 1], sin[start:start + 1], FA).transpose(1, 0, 2)
            q, k = rot(q), rot(k)
        ck = np.concatenate((ck, np.transpose(k, (1, 0, 2))), axis=1)
        cv = np.concatenate((cv, np.transpose(v, (1, 0, 2))), axis=1)
        attended = o.attention_cached(q, ck, cv, start, heads, n_kv, FA, window)
        ref = lin(oraw, o.Q6_K, attended, d_model, q_nb)
        got = bank.apply(0, qh, kh, vh, oh, x, FW, window, rope)
        assert np.array_equal(got, ref), (rope, window)
        start += 1
        assert bank.length(0) == start
    # the bank is full after max_length rows
    bank.apply(0, qh, kh, vh, oh, probe, FW, None, False)
    assert bank.length(0) == max_length
    with pytest.raises(ValueError, match="already holds its"):
        bank.apply(0, qh, kh, vh, oh, probe, FW, None, False)
    bank.reset()
    assert bank.length(0) == 0
    bank.close()
    bank.close()                                           # idempotent request cleanup

    # rows the bank cannot hold exactly fail loudly at the next apply and poison the layer
    bad = qk_cuda.ResidentAttentionCache(1, max_length, d_model, heads, n_kv, head_dim, FA, cos, sin)
    bad.import_layer(0, np.zeros((n_kv, 1, head_dim), dtype=np.int64),
                     np.full((n_kv, 1, head_dim), np.iinfo(np.int64).max, dtype=np.int64))
    with pytest.raises(qk_cuda.CudaContextError, match="left the exact envelope"):
        bad.apply(0, qh, kh, vh, oh, probe, FW, None, False)
    with pytest.raises(qk_cuda.CudaContextError, match="native status"):
        bad.apply(0, qh, kh, vh, oh, probe, FW, None, False)
    bad.close()
    qk_cuda.free_all()


def test_bank_rejects_bad_dimensions():
    cos, sin = o.build_rope_tables(4, 64, 50000.0, FA)
    with pytest.raises(ValueError):
        qk_cuda.ResidentAttentionCache(1, 4, 300, 4, 2, 64, FA, cos, sin)
    with pytest.raises(ValueError):
        qk_cuda.ResidentAttentionCache(1, 5, 256, 4, 2, 64, FA, cos, sin)            # table rows != max_length
    lib = qk_cuda.load_library()
    assert lib.qk_attention_bank_reset(12345) == 1
    assert lib.qk_attention_bank_import(12345, 0, None, None, 0) == 1
