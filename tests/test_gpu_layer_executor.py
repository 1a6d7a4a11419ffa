"""GPU parity of the retained-layer executor (qk_attention_bank_moe_configure / bind / begin / continue / export and the
executor class over them): a token walks consecutive MoE layers with its residual row, routing and attention row kept on
the device, only the ids of unbound experts come back, and the published row equals the host composition
    x + attention(rmsnorm(x)) + moe(rmsnorm(x))
of every layer, byte for byte.  Mirrors the reference's own gate for this protocol
(north-mini-code/tests/test_qk_cuda.py::test_cuda_resident_moe_layer_cold_continuation_retains_exact_residual)."""
import numpy as np
import pytest

from integer_inference_engine_b200 import qk_cuda
from oracle import native as onat
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FA, FW = 16, 24
D, HEADS, N_KV, HD = 256, 8, 2, 64
EXPERTS, USED, E_FFN, ROWS = 6, 2, 256, 4


class Case:
    def __init__(self, down_q=o.Q6_K):
        rng = np.random.default_rng(515)
        self.nb, self.qw = D // 256, HEADS * HD
        mk = lambda out_f, qt, seed, nb=D // 256: (o.synth_q4k if qt == o.Q4_K else o.synth_q6k)(np.random.default_rng(seed), out_f, nb)
        self.raw = {"q": (mk(self.qw, o.Q4_K, 1), self.qw, self.nb, o.Q4_K), "k": (mk(N_KV * HD, o.Q6_K, 2), N_KV * HD, self.nb, o.Q6_K),
                    "v": (mk(N_KV * HD, o.Q4_K, 3), N_KV * HD, self.nb, o.Q4_K), "o": (mk(D, o.Q6_K, 4, self.qw // 256), D, self.qw // 256, o.Q6_K)}
        self.h = {name: qk_cuda.register_weight(*spec) for name, spec in self.raw.items()}
        self.gain = rng.integers(1 << 15, 1 << 17, size=D, dtype=np.int64)
        self.router = rng.integers(-(1 << 13), 1 << 13, size=(EXPERTS, D), dtype=np.int64)
        self.gain_h, self.router_h = qk_cuda.register_i64(self.gain), qk_cuda.register_i64(self.router)
        self.down_q = down_q
        self.gate = [mk(E_FFN, o.Q4_K, 100 + e) for e in range(EXPERTS)]
        self.up = [mk(E_FFN, o.Q4_K, 200 + e) for e in range(EXPERTS)]
        self.down = [mk(D, down_q, 300 + e, E_FFN // 256) for e in range(EXPERTS)]
        self.loaded = {}
        self.cos, self.sin = o.build_rope_tables(ROWS, HD, 50000.0, FA)
        self.kv = {}                                        # layer -> (K rows, V rows) of the host composition

    def load(self, expert):
        if expert not in self.loaded:
            self.loaded[expert] = (qk_cuda.register_weight(self.gate[expert], E_FFN, self.nb, o.Q4_K),
                                   qk_cuda.register_weight(self.up[expert], E_FFN, self.nb, o.Q4_K),
                                   qk_cuda.register_weight(self.down[expert], D, E_FFN // 256, self.down_q))
        return self.loaded[expert]

    def lin(self, name, x):
        raw, out_f, nb, qt = self.raw[name]
        return onat.qk_linear(raw, x, out_f, nb, FW, qt)

    def host_layer(self, layer, x, rope, window, router=None):
        """(selected ids, x + attention + moe) of one token on the host, advancing the host K/V rows of ``layer``."""
        router = self.router if router is None else router
        h = o.rmsnorm_fixed(x, FA, 1, self.gain)
        logits = o.linear(h, router, FW)[0]
        ids = o.topk_lowidx(logits, USED)
        gates = o.sigmoid_fixed(logits[ids].astype(np.int64), FA)
        ck, cv = self.kv.get(layer, (np.zeros((N_KV, 0, HD), np.int64), np.zeros((N_KV, 0, HD), np.int64)))
        pos = ck.shape[1]
        q = self.lin("q", h).reshape(1, HEADS, HD)
        k = self.lin("k", h).reshape(1, N_KV, HD)
        v = self.lin("v", h).reshape(1, N_KV, HD)
        if rope:
            rot = lambda t: o.rope_fixed(np.transpose(t, (1, 0, 2)), self.cos[pos:pos + 1], self.sin[pos:pos + 1], FA).transpose(1, 0, 2)
            q, k = rot(q), rot(k)
        ck = np.concatenate((ck, np.transpose(k, (1, 0, 2))), axis=1)
        cv = np.concatenate((cv, np.transpose(v, (1, 0, 2))), axis=1)
        self.kv[layer] = (ck, cv)
        attention = self.lin("o", o.attention_cached(q, ck, cv, pos, HEADS, N_KV, FA, window))
        moe = np.zeros(D, dtype=np.int64)
        for slot, e in enumerate(ids):
            g = onat.qk_linear(self.gate[e], h, E_FFN, self.nb, FW, o.Q4_K)
            u = onat.qk_linear(self.up[e], h, E_FFN, self.nb, FW, o.Q4_K)
            gu = o.mul_shift(o.silu_int(g, FA), u, FA)
            dn = onat.qk_linear(self.down[e], gu, D, E_FFN // 256, FW, self.down_q)[0]
            moe = moe + o.mul_shift(dn, np.int64(gates[slot]), FA)
        return [int(e) for e in ids], np.asarray(x, np.int64) + attention + moe[None]


def _oracle_names():
    need = ("rmsnorm_fixed", "linear", "topk_lowidx", "sigmoid_fixed", "silu_int", "mul_shift", "attention_cached", "rope_fixed")
    return [n for n in need if not hasattr(o, n)]


def test_oracle_has_the_pieces():
    assert _oracle_names() == []


@pytest.mark.parametrize("down_q", (o.Q6_K, o.Q4_K), ids=("down-q6k", "down-q4k"))
def test_cold_continuation_keeps_the_exact_residual(down_q):
    qk_cuda.free_all()
    c = Case(down_q)
    rng = np.random.default_rng(77)
    bank = qk_cuda.ResidentAttentionCache(2, ROWS, D, HEADS, N_KV, HD, FA, c.cos, c.sin)
    for layer in range(2):
        bank.configure_moe_layer(layer, EXPERTS, USED, D, E_FFN)
    bank.configure_moe_layer(0, EXPERTS, USED, D, E_FFN)                  # same shape again: accepted
    with pytest.raises(ValueError, match="already configured"):
        bank.configure_moe_layer(0, EXPERTS, 1, D, E_FFN)
    x0 = rng.integers(-(1 << 17), 1 << 17, size=(1, D), dtype=np.int64)
    ids0, ref0 = c.host_layer(0, x0, True, 3)
    bank.bind_moe_expert(0, ids0[0], *c.load(ids0[0]))
    args = (c.gain_h, c.router_h, c.h["q"], c.h["k"], c.h["v"], c.h["o"])
    # a projection handle of the wrong kind is refused before anything moves
    with pytest.raises(qk_cuda.CudaContextError, match="native status 1"):
        bank.begin_moe_layer(0, c.gain_h, c.router_h, c.gain_h, c.h["k"], c.h["v"], c.h["o"], x0, FW, 1, 3, True)
    assert bank.length(0) == 0
    before = qk_cuda.resident_count()
    qk_cuda.profile_reset(enabled=True)
    cold = bank.begin_moe_layer(0, *args, x0, FW, 1, 3, True)
    assert cold == (ids0[1],)
    assert qk_cuda.resident_count() == before                             # finding the cold set uploads nothing
    stats = qk_cuda.profile_snapshot()
    assert stats["d2h_calls"] == 2 and stats["d2h_bytes"] == 4 + 4 * (USED + 1)
    with pytest.raises(qk_cuda.CudaContextError, match="remain unbound"):
        bank.continue_moe_layer(0, FW)
    with pytest.raises(qk_cuda.CudaContextError):                         # nothing else runs on the bank while a layer is pending
        bank.apply(1, c.h["q"], c.h["k"], c.h["v"], c.h["o"], x0, FW, None, False)
    bank.bind_moe_expert(0, cold[0], *c.load(cold[0]))
    kept = bank.continue_moe_layer(0, FW)
    assert isinstance(kept, qk_cuda.ResidentLayerHidden)
    assert np.array_equal(bank.export_moe_hidden(), ref0)

    ids1, ref1 = c.host_layer(1, ref0, False, None)
    for e in ids1:
        if e in c.loaded:
            bank.bind_moe_expert(1, e, *c.loaded[e])
    cold1 = bank.begin_moe_layer(1, *args, kept, FW, 1, None, False)
    assert cold1 == tuple(e for e in ids1 if e not in c.loaded)
    for e in cold1:
        bank.bind_moe_expert(1, e, *c.load(e))
    got = bank.continue_moe_layer(1, FW, publish=True)
    assert np.array_equal(got, ref1)
    assert np.array_equal(bank.export_moe_hidden(), ref1)
    with pytest.raises(ValueError, match="stale"):                        # the marker of layer 0 is no longer the retained row
        bank.begin_moe_layer(0, *args, kept, FW, 1, 3, True)
    qk_cuda.profile_set_enabled(False)
    bank.close()
    qk_cuda.free_all()


def test_executor_chain_second_token_allocates_nothing():
    qk_cuda.free_all()
    c = Case()
    rng = np.random.default_rng(78)
    layers = 3
    tied = np.zeros_like(c.router)                                        # all logits tie: experts 0 and 1 every time
    tied_h = qk_cuda.register_i64(tied)
    bank = qk_cuda.ResidentAttentionCache(layers, ROWS, D, HEADS, N_KV, HD, FA, c.cos, c.sin)
    loads = []

    def load(layer, expert):
        loads.append((layer, expert))
        return c.load(expert)

    ex = qk_cuda.ResidentMoeTokenExecutor(bank, first_layer=0, layer_count=layers, n_experts=EXPERTS, n_used=USED, d_model=D,
                                          expert_ffn=E_FFN, fw=FW, eps=1, lookup_expert=lambda _l, e: c.loaded.get(e), load_expert=load)
    specs = [qk_cuda.ResidentMoeLayerSpec(l, c.gain_h, tied_h, c.h["q"], c.h["k"], c.h["v"], c.h["o"], None if l % 2 else 3, l % 2 == 0)
             for l in range(layers)]
    empty = bank.workspace_bytes()
    qk_cuda.profile_reset(enabled=True)
    for token in range(2):
        x = rng.integers(-(1 << 17), 1 << 17, size=(1, D), dtype=np.int64)
        ref = x
        for l in range(layers):
            ids, ref = c.host_layer(l, ref, l % 2 == 0, None if l % 2 else 3, tied)
            assert ids == [0, 1]
        if token == 1:
            first = qk_cuda.profile_snapshot()
            warm = bank.workspace_bytes()
            assert warm > empty and first["allocation_calls"] > 0
        got = ex.run(x, specs)
        assert np.array_equal(got, ref), token
    second = qk_cuda.profile_snapshot()
    assert loads == [(l, e) for l in range(layers) for e in (0, 1)]       # only the first token found cold experts
    assert second["allocation_calls"] == first["allocation_calls"]
    assert second["d2h_calls"] - first["d2h_calls"] == 3 * layers + 1     # per layer two flag words and the cold list; one row out
    assert bank.workspace_bytes() == warm
    qk_cuda.profile_set_enabled(False)

    # an input outside the norm's envelope raises the guard, appends nothing and leaves the layer unusable
    bad = qk_cuda.ResidentAttentionCache(1, ROWS, D, HEADS, N_KV, HD, FA, c.cos, c.sin)
    bad.configure_moe_layer(0, EXPERTS, USED, D, E_FFN)
    unsafe = np.zeros((1, D), dtype=np.int64)
    unsafe[0, :2] = np.iinfo(np.int64).min
    with pytest.raises(qk_cuda.CudaContextError, match="left the exact envelope"):
        bad.begin_moe_layer(0, c.gain_h, c.router_h, c.h["q"], c.h["k"], c.h["v"], c.h["o"], unsafe, FW, 1, None, False)
    assert bad.length(0) == 0
    with pytest.raises(qk_cuda.CudaContextError, match="native status 1"):
        bad.begin_moe_layer(0, c.gain_h, c.router_h, c.h["q"], c.h["k"], c.h["v"], c.h["o"], np.zeros((1, D), np.int64), FW, 1, None, False)
    bad.close()
    bank.close()
    qk_cuda.free_all()
