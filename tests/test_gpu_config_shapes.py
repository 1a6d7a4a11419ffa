"""GPU parity at the benchmark's exact shapes.

Config 1: one integer MoE block, seed 0, d = 2048, 128 experts, top-8, expert width 768, 16 tokens, against the
golden ids / output bytes recorded from the reference's own ``moe_layer_int`` (tests/golden/moe.npz, "config1"),
through the device front end and through the reference-facing host entry ``qk_moe_ffn_batched``.
Config 3: 2048 tokens through the same block shape (grouped expert GEMMs on tcgen05), sampled rows against the C
oracle, with the tensor-core tile shape that served each stage checked by its launch counter.
"""
import numpy as np
import pytest

from oracle import native as onat
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FA, FW = 16, 24
D, EFF, E, K = 2048, 768, 128, 8


def _register(qk, router, gate, up, down, d=D, eff=EFF):
    rh = qk.register_weight(router, len(gate), d // 256, o.Q4_K)
    gh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in gate]
    uh = [qk.register_weight(w, eff, d // 256, o.Q4_K) for w in up]
    dh = [qk.register_weight(w, d, eff // 256, o.Q6_K) for w in down]
    return rh, gh, uh, dh


def _oracle_rows(router, gate, up, down, h_rows, k, d=D, eff=EFF):
    """C-oracle routing, gates and block output of a few rows (rows are independent in the MoE block)."""
    return onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, k, h_rows, d, eff, FA, FW)


def test_config1_block_equals_the_reference_golden(golden_dir):
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    qk.free_all()
    seed, d, eff, n_e, k, T = o.GOLDEN_MOE_CASES["config1"]
    assert (seed, d, eff, n_e, k, T) == (0, D, EFF, E, K, 16)
    g = np.load(golden_dir / "moe.npz")
    router, gate, up, down, h = o.synth_moe(seed, d, eff, n_e, T)
    rh, gh, uh, dh = _register(qk, router, gate, up, down)
    # (a) device front end: routing + experts on the device
    layer = device.MoELayer(rh, gh, uh, dh, k, d, eff)
    out, ids, gates = layer.forward(torch.from_numpy(h).cuda(), FA, FW)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(ids.cpu().numpy(), g["config1_ids"]), "router indices differ from the reference"
    assert np.array_equal(out.cpu().numpy(), g["config1_out"]), "block output bytes differ from the reference"
    # (b) the reference's own host entry: handles flattened token-major, gates from the routed logits
    sel = g["config1_ids"]
    logits = onat.qk_linear(router, h, n_e, d // 256, FW, o.Q4_K)
    gts = np.stack([onat.sigmoid(logits[t][sel[t]], FA) for t in range(T)])
    assert np.array_equal(gates.cpu().numpy(), gts)
    flat = lambda hs: [hs[e] for t in range(T) for e in sel[t]]
    for dp4a in (False, True):
        got = qk.moe_ffn_batched(flat(gh), flat(uh), flat(dh), T, k, h, gts.reshape(-1), d, eff, FA, FW, dp4a=dp4a)
        assert got is not None and np.array_equal(got, g["config1_out"]), f"qk_moe_ffn_batched (dp4a={dp4a})"
    # one token at a time through the decode entry
    for t in (0, 15):
        got = qk.moe_ffn([gh[e] for e in sel[t]], [uh[e] for e in sel[t]], [dh[e] for e in sel[t]], h[t], gts[t], d, eff, FA, FW)
        assert np.array_equal(got, g["config1_out"][t])
    qk.free_all()


@pytest.fixture(scope="module")
def config3_block():
    """The config-1 block (seed 0) registered once, with 2048 rows of to_fixed(N(0,1)) as the prefill input."""
    from integer_inference_engine_b200 import qk_cuda as qk
    qk.free_all()
    router, gate, up, down, _ = o.synth_moe(0, D, EFF, E, 1)
    handles = _register(qk, router, gate, up, down)
    h = o.to_fixed(np.random.default_rng(3).standard_normal((2048, D)), FA)
    yield (router, gate, up, down), handles, h
    qk.free_all()


# name -> (multiplier of the hidden rows, expected gate/up tile shape, expected down tile shape or None when the product
# needs more digits than a tile carries); shapes are indices of iie_prefill_launch_counts
CONFIG3_CASES = {"config3": (1, 0, 2), "gu_six_digits": (16, 0, 3), "h_four_digits": (200, 1, None)}


@pytest.mark.parametrize("name", list(CONFIG3_CASES))
def test_config3_prefill_shape_on_tensor_cores(config3_block, name):
    import torch

    from integer_inference_engine_b200 import device
    (router, gate, up, down), (rh, gh, uh, dh), h = config3_block
    mult, want_gu, want_dn = CONFIG3_CASES[name]
    T = 2048 if name == "config3" else 512
    h = h[:T] * mult
    layer = device.MoELayer(rh, gh, uh, dh, K, D, EFF)
    before = device.prefill_launch_counts()
    out, ids, gates = layer.forward(torch.from_numpy(h).cuda(), FA, FW)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    delta = [b - a for a, b in zip(before, device.prefill_launch_counts())]
    assert delta[5] + delta[6] == 1, f"router product not on the tensor-core tiles: {delta}"
    assert delta[want_gu] == 1 and delta[0] + delta[1] == 1, f"gate/up tile shape: {delta}"
    if want_dn is None:
        assert delta[2] + delta[3] + delta[4] == 0, f"down stage should have streamed: {delta}"
    else:
        assert delta[want_dn] == 1 and delta[2] + delta[3] == 1, f"down tile shape: {delta}"
    rows = np.unique(np.concatenate([np.arange(0, T, max(1, T // 60)), [T - 1, T - 2, 1, 2]]))
    assert len(rows) >= 64 or T < 2048
    ids_ref, gates_ref, out_ref = _oracle_rows(router, gate, up, down, h[rows], K)
    assert np.array_equal(ids.cpu().numpy()[rows], ids_ref)
    assert np.array_equal(gates.cpu().numpy()[rows], gates_ref)
    assert np.array_equal(out.cpu().numpy()[rows], out_ref)
    counts = np.bincount(ids.cpu().numpy().reshape(-1), minlength=E)
    assert counts.sum() == T * K                       # every (token, slot) pair was dispatched to exactly one expert
    layer.close()


def test_reference_prefill_entry_reaches_the_tensor_cores(config3_block):
    """m = 256, k = 8 through ``qk_moe_ffn_batched`` (what Engine._moe calls for a prefill, engine.py:389-411): the
    grouped tcgen05 tiles serve it and the bytes equal the oracle's."""
    from integer_inference_engine_b200 import device, qk_cuda as qk
    (router, gate, up, down), (rh, gh, uh, dh), h = config3_block
    m = 256
    h = h[1000:1000 + m]
    ids_ref, gates_ref, out_ref = _oracle_rows(router, gate, up, down, h, K)
    flat = lambda hs: [hs[e] for t in range(m) for e in ids_ref[t]]
    before = device.prefill_launch_counts()
    got = qk.moe_ffn_batched(flat(gh), flat(uh), flat(dh), m, K, h, gates_ref.reshape(-1), D, EFF, FA, FW)
    delta = [b - a for a, b in zip(before, device.prefill_launch_counts())]
    assert delta[0] == 1 and delta[2] + delta[3] == 1, f"prefill-sized host call did not launch the tensor-core tiles: {delta}"
    assert got is not None and np.array_equal(got, out_ref)
    # a token may be handed experts other than its own routing: token 1 gets token 0's experts with its own gates
    gl, ul, dl = flat(gh), flat(uh), flat(dh)
    gl[8:16], ul[8:16], dl[8:16] = gl[0:8], ul[0:8], dl[0:8]
    got2 = qk.moe_ffn_batched(gl, ul, dl, m, K, h, gates_ref.reshape(-1), D, EFF, FA, FW)
    want1 = np.zeros(D, dtype=object)
    for j, e in enumerate(ids_ref[0]):
        g_ = onat.silu(onat.qk_linear(gate[e], h[1:2], EFF, D // 256, FW, o.Q4_K), FA)
        u_ = onat.qk_linear(up[e], h[1:2], EFF, D // 256, FW, o.Q4_K)
        dn = onat.qk_linear(down[e], o.mul_shift(g_, u_, FA), D, EFF // 256, FW, o.Q6_K)[0].astype(object)
        want1 += (dn * int(gates_ref[1, j])) >> FA
    assert np.array_equal(got2[1], want1.astype(np.int64)) and np.array_equal(got2[2:], out_ref[2:])
