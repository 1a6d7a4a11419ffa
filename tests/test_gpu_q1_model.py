"""GPU parity of the 1-bit decoder's whole decode token (Q1_0 embedding row -> sequential attention / SwiGLU
blocks -> Q1_0 head -> greedy pick): the reference's own recorded step, then seeded synthetic decoders against
the CPU checker, eager and as a replayed CUDA graph; and the two element-wise entries it adds."""
import numpy as np
import pytest

from oracle import model_oracle
from oracle import qk_oracle as o
from test_oracle_golden import q1_golden_layers

pytestmark = pytest.mark.gpu
FRAC = 16


@pytest.fixture(scope="module", autouse=True)
def _library():
    from integer_inference_engine_b200 import q1_gpu, qk_cuda
    assert q1_gpu.gpu_available(), "the CUDA library must be built and a GPU present"
    yield
    q1_gpu.q1_free_weights()
    qk_cuda.free_all()


def test_swiglu_wraps_like_numpy():
    import torch

    from integer_inference_engine_b200 import q1_gpu
    rng = np.random.default_rng(5)
    gate = rng.integers(-(1 << 22), 1 << 22, size=4096, dtype=np.int64)
    up = rng.integers(-(1 << 22), 1 << 22, size=4096, dtype=np.int64)
    edge = np.array([np.iinfo(np.int64).min, np.iinfo(np.int64).max, -1, 0, 1, 1 << 62, -(1 << 62), 1 << 40, -(1 << 40)], np.int64)
    gate[:9], up[:9] = edge, edge[::-1]
    gate[9:18], up[9:18] = edge, 3 << 45
    got = q1_gpu.silu_mul_dev(torch.from_numpy(gate).cuda(), torch.from_numpy(up).cuda(), FRAC).cpu().numpy()
    assert np.array_equal(got, model_oracle.q1_swiglu(gate, up, FRAC))


@pytest.mark.parametrize("wide", [False, True])
def test_embedding_rows(wide):
    import torch

    from integer_inference_engine_b200 import q1_gpu
    rng = np.random.default_rng(6 + wide)
    bits, scale = o.synth_q1(rng, 70, 3)
    if wide:
        scale = rng.integers(-(1 << 40), 1 << 40, size=scale.shape, dtype=np.int64)
    else:
        scale = scale.astype(np.int32)
    h = q1_gpu.q1_register_weight(bits, scale)
    out = torch.empty(3 * 128, dtype=torch.int64, device="cuda")
    cell = torch.zeros(1, dtype=torch.int32, device="cuda")
    for row in (0, 1, 15, 16, 37, 69):
        want = model_oracle.q1_rows(bits, scale, row)[0]
        assert np.array_equal(q1_gpu.embed_dev(h, row, out).cpu().numpy(), want)
        cell.fill_(row)
        assert np.array_equal(q1_gpu.embed_dev(h, cell, out).cpu().numpy(), want)
    with pytest.raises(RuntimeError):
        q1_gpu.embed_dev(h, 70, out)


def test_recorded_reference_step(golden_dir):
    import torch

    from integer_inference_engine_b200 import device
    from integer_inference_engine_b200.q1_model import Q1Decoder
    g = np.load(golden_dir / "q1_decode.npz")
    layers, top, cfg = q1_golden_layers(g, rows=8)
    pos = int(g["pos"])
    m = Q1Decoder(cfg["d"], cfg["H"], cfg["Hkv"], cfg["hd"], cfg["ffn"], 96, layers, top, g["cos"], g["sin"], pos, FRAC)
    m.token.fill_(int(g["token"]))
    device.read_flags()
    m.step(pos)
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    assert np.array_equal(m.x.cpu().numpy(), g["x"])
    assert np.array_equal(m.logits.cpu().numpy(), g["logits"]) and int(m.token.item()) == int(g["next"])
    for li in range(2):
        assert np.array_equal(m.layers[li]["k"][:, :pos + 1].cpu().numpy(), g[f"k{li}_after"])
        assert np.array_equal(m.layers[li]["v"][:, :pos + 1].cpu().numpy(), g[f"v{li}_after"])


def test_decode_steps_match_the_checker_eager_and_replayed():
    import torch

    from integer_inference_engine_b200 import device
    from integer_inference_engine_b200.q1_model import SyntheticQ1Decoder
    m = SyntheticQ1Decoder(n_layers=3, d_model=512, n_heads=8, n_kv=4, head_dim=64, d_ffn=768, vocab=1000, context=30,
                           max_new=8, seed=11, keep_host=True)
    layers = [dict(L, k=L["k"].cpu().numpy().astype(np.int64), v=L["v"].cpu().numpy().astype(np.int64)) for L in m.host_layers]
    cfg = dict(d=m.d, H=m.H, Hkv=m.Hkv, hd=m.hd, ffn=m.ffn, frac=FRAC)
    cos, sin = m.cos.cpu().numpy(), m.sin.cpu().numpy()
    token, pos = 123, m.context
    m.token.fill_(token)
    device.read_flags()
    for step in range(5):
        if step == 2:
            m.capture(m.context + 7)
        want, trace, logits = model_oracle.q1_decode_token(token, pos, layers, m.host_top, cfg, cos, sin)
        if step < 2:
            m.step(pos)
        else:
            m.replay()
        torch.cuda.synchronize()
        assert device.read_flags() == 0
        assert np.array_equal(m.x.cpu().numpy(), trace[-1:]), step
        assert np.array_equal(m.logits.cpu().numpy()[0], logits), step
        assert int(m.token.item()) == want and int(m.pos.item()) == pos + 1
        for li in range(m.n_layers):
            assert np.array_equal(m.layers[li]["k"][:, pos].cpu().numpy(), layers[li]["k"][:, pos]), (step, li)
        token, pos = want, pos + 1


@pytest.mark.parametrize(("T", "nb"), [(1, 4), (3, 4), (1, 9), (2, 32)])
def test_fused_product_forms(T, nb):
    """Norm, SwiGLU and residual steps folded into the product's launches against their separate restatements."""
    import torch

    from integer_inference_engine_b200 import device, q1_gpu
    from oracle import native as onat
    rng = np.random.default_rng(40 + T + nb)
    out_f = 200
    K = nb * 128
    bits, scale = o.synth_q1(rng, out_f, nb)
    h = q1_gpu.q1_register_weight(bits, scale.astype(np.int32))
    x = o.to_fixed(rng.standard_normal((T, K)) * 3, FRAC)
    gain = np.rint((np.abs(rng.standard_normal(K)) + 0.5) * (1 << FRAC)).astype(np.int64)
    res = rng.integers(-(1 << 40), 1 << 40, size=(T, out_f), dtype=np.int64)
    cuda = lambda a: torch.from_numpy(a).cuda()
    device.read_flags()
    out = torch.empty((T, out_f), dtype=torch.int64, device="cuda")
    # plain, with a residual that is the output buffer itself
    out.copy_(cuda(res))
    q1_gpu.apply_fused_dev(h, cuda(x), FRAC, out, add=out)
    assert np.array_equal(out.cpu().numpy(), onat.q1_linear(x, bits, scale, FRAC) + res)
    # RMSNorm with and without a gain
    for g in (gain, None):
        q1_gpu.apply_fused_dev(h, cuda(x), FRAC, out, norm=True, gain=None if g is None else cuda(g))
        assert np.array_equal(out.cpu().numpy(), onat.q1_linear(o.rmsnorm_fixed(x, FRAC, 1, g), bits, scale, FRAC))
    # SwiGLU of two column slices of one buffer, plus a residual
    gu = rng.integers(-(1 << 21), 1 << 21, size=(T, 2 * K), dtype=np.int64)
    gu[0, :4] = [np.iinfo(np.int64).min, np.iinfo(np.int64).max, 1 << 50, -(1 << 50)]
    gud = cuda(gu)
    q1_gpu.apply_fused_dev(h, gud[:, :K], FRAC, out, up=gud[:, K:], add=cuda(res))
    with np.errstate(over="ignore"):
        want = onat.q1_linear(model_oracle.q1_swiglu(gu[:, :K], gu[:, K:], FRAC), bits, scale, FRAC) + res
    assert np.array_equal(out.cpu().numpy(), want)
    assert device.read_flags() == 0
    # a row outside the RMSNorm envelope raises the flag instead of a wrong value
    big = x.copy(); big[0, 0] = 1 << 60
    q1_gpu.apply_fused_dev(h, cuda(big), FRAC, out, norm=True, gain=cuda(gain))
    torch.cuda.synchronize()
    assert device.read_flags() & 2


def test_head_norms_in_one_launch():
    import torch

    from integer_inference_engine_b200 import device, q1_gpu
    rng = np.random.default_rng(50)
    H, Hkv, hd = 8, 2, 64
    x = o.to_fixed(rng.standard_normal((H + Hkv, hd)) * 5, FRAC)
    ga = np.rint((np.abs(rng.standard_normal(hd)) + 0.5) * (1 << FRAC)).astype(np.int64)
    gb = np.rint((np.abs(rng.standard_normal(hd)) + 0.5) * (1 << FRAC)).astype(np.int64)
    out = torch.empty((H + Hkv, hd), dtype=torch.int64, device="cuda")
    device.read_flags()
    q1_gpu.head_norm_dev(torch.from_numpy(x).cuda(), H, Hkv, hd, torch.from_numpy(ga).cuda(), torch.from_numpy(gb).cuda(), FRAC, out)
    want = np.concatenate([o.rmsnorm_fixed(x[:H], FRAC, 1, ga), o.rmsnorm_fixed(x[H:], FRAC, 1, gb)])
    assert np.array_equal(out.cpu().numpy(), want) and device.read_flags() == 0


@pytest.mark.parametrize(("rows", "width"), [(1, 4096), (3, 1536), (1, 1000), (20, 2048)])
def test_rmsnorm_long_rows(rows, width):
    """Long rows are normalised by several CTAs each; values beyond the narrow-division range take the wide path."""
    import torch

    from integer_inference_engine_b200 import device, qk_cuda
    rng = np.random.default_rng(60 + rows + width)
    x = o.to_fixed(rng.standard_normal((rows, width)) * 4, FRAC)
    x[0, 1] = 1 << 50; x[-1, width - 1] = -(1 << 49) - 12345
    gain = np.rint((np.abs(rng.standard_normal(width)) + 0.5) * (1 << FRAC)).astype(np.int64)
    gh = qk_cuda.register_i64(gain)
    device.read_flags()
    for g, h in ((gain, gh), (None, -1)):
        got = device.rmsnorm(torch.from_numpy(x).cuda(), h, FRAC, 1).cpu().numpy()
        assert np.array_equal(got, o.rmsnorm_fixed(x, FRAC, 1, g))
    assert device.read_flags() == 0


@pytest.mark.parametrize(("out_f", "nb"), [(48, 1), (200, 4), (4096, 32), (1000, 96), (33, 128)])
def test_single_token_launch_forms_agree(out_f, nb):
    """The bulk-copy kernel and the per-lane-load kernel against the checker, int32 and int64 scales."""
    import torch

    from integer_inference_engine_b200 import device, q1_gpu
    from oracle import native as onat
    rng = np.random.default_rng(70 + out_f + nb)
    bits, scale = o.synth_q1(rng, out_f, nb)
    x = rng.integers(-(1 << 40), 1 << 40, size=(1, nb * 128), dtype=np.int64)
    xd = torch.from_numpy(x).cuda()
    device.read_flags()
    try:
        for sc in (scale.astype(np.int32), rng.integers(-(1 << 40), 1 << 40, size=scale.shape, dtype=np.int64)):
            h = q1_gpu.q1_register_weight(bits, sc)
            want = onat.q1_linear(x, bits, sc.astype(np.int64), FRAC)
            for form in (True, False):
                q1_gpu.set_stream_form(form)
                assert np.array_equal(q1_gpu.apply_dev(h, xd, FRAC).cpu().numpy(), want), (form, sc.dtype)
    finally:
        q1_gpu.set_stream_form(False)
    assert device.read_flags() == 0
