"""GPU parity of the Q1_0 dense path through the C-ABI (the reference's own entry names) against the
golden vectors generated from the reference and against the CPU oracle."""
import numpy as np
import pytest

from integer_inference_engine_b200 import q1_gpu
from oracle import native as onat
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
FRAC = 16


@pytest.fixture(scope="module", autouse=True)
def _library():
    assert q1_gpu.gpu_available(), "the CUDA library must be built and a GPU present"
    yield
    q1_gpu.q1_free_weights()


def _case(seed, out_f, nb, T, magbits, wide_scale=False):
    rng = np.random.default_rng(seed)
    bits, scale = o.synth_q1(rng, out_f, nb)
    if wide_scale:
        scale = rng.integers(-(1 << 40), 1 << 40, size=scale.shape, dtype=np.int64)
    x = rng.integers(-(1 << magbits), 1 << magbits, size=(T, nb * 128), dtype=np.int64)
    return bits, scale, x


def test_golden_vectors_from_the_reference(golden_dir):
    """Same seeds as tests/golden/make_golden.py; y_* are reference_bonsai.q1_linear_ref outputs."""
    g = np.load(golden_dir / "q1.npz")
    for i, (out_f, nb, T, magbits) in enumerate([(7, 3, 1, 20), (7, 3, 3, 20), (16, 2, 2, 62)]):
        bits, scale, x = _case(500 + i, out_f, nb, T, magbits, wide_scale=magbits > 40)
        assert np.array_equal(q1_gpu.q1_apply_gpu(x, bits, scale, FRAC), g[f"y_{i}"])
        assert np.array_equal(q1_gpu.q1_apply_dp4a_gpu(x, bits, scale, FRAC, L=8), g[f"y_{i}"])


@pytest.mark.parametrize("out_f,nb,T", [(16, 1, 1), (33, 5, 1), (256, 32, 1), (4096, 32, 1), (512, 96, 1), (48, 130, 1),
                                        (16, 1, 2), (100, 7, 5), (256, 32, 33), (64, 96, 70), (1024, 32, 4), (200, 3, 129), (130, 1, 64), (9, 2, 32)])
def test_linear_matches_the_oracle(out_f, nb, T):
    bits, scale, x = _case(out_f * 131 + nb * 7 + T, out_f, nb, T, 26)
    want = onat.q1_linear(x, bits, scale, FRAC)
    assert np.array_equal(q1_gpu.q1_apply_gpu(x, bits, scale, FRAC), want)


@pytest.mark.parametrize("magbits", [8, 31, 40, 55, 63])
@pytest.mark.parametrize("T", [1, 6, 40])
def test_every_int64_activation_is_exact(magbits, T):
    """Sums wrap modulo 2^64 exactly as in the reference, including the int64 extremes."""
    bits, scale, x = _case(900 + magbits + T, 40, 4, T, magbits, wide_scale=True)
    x[0, :4] = [np.iinfo(np.int64).min, np.iinfo(np.int64).max, -1, 0]
    want = onat.q1_linear(x, bits, scale, FRAC)
    assert np.array_equal(q1_gpu.q1_apply_gpu(x, bits, scale, FRAC), want)


@pytest.mark.parametrize("frac", [0, 1, 16, 30, 62, 63])
def test_shift_amounts(frac):
    bits, scale, x = _case(77 + frac, 24, 3, 3, 30)
    scale = -scale if frac % 2 else scale                          # negative products exercise the floor
    want = onat.q1_linear(x, bits, scale, frac)
    assert np.array_equal(q1_gpu.q1_apply_gpu(x, bits, scale, frac), want)


def test_all_set_and_all_clear_bits():
    _, scale, x = _case(5, 16, 2, 2, 20)
    for fill in (0x00, 0xFF):
        bits = np.full((16, 2, 16), fill, np.uint8)
        assert np.array_equal(q1_gpu.q1_apply_gpu(x, bits, scale, FRAC), onat.q1_linear(x, bits, scale, FRAC))


def test_resident_weights_int64_and_int32_scales():
    bits, scale, x = _case(11, 200, 8, 3, 24)
    want = onat.q1_linear(x, bits, scale, FRAC)
    before = q1_gpu.gpu_memory_info()["resident_weight_bytes"]
    h64 = q1_gpu.q1_register_weight(bits, scale)
    h32 = q1_gpu.q1_register_weight(bits, scale.astype(np.int32))
    hco = q1_gpu.q1_register_weight(bits, scale.astype(np.int32), gpu_coalesced=True)
    hbm = q1_gpu.q1_register_weight(bits, scale.astype(np.int32), gpu_bmma=True)
    assert len({h64, h32, hco, hbm}) == 4
    after = q1_gpu.gpu_memory_info()["resident_weight_bytes"]
    assert after - before == bits.size * 4 + scale.size * (8 + 4 * 3)
    for h in (h64, h32, hco, hbm):
        assert np.array_equal(q1_gpu.q1_apply_resident(h, x, 200, 8, FRAC), want)
        assert np.array_equal(q1_gpu.q1_apply_resident(h, x[:1], 200, 8, FRAC), want[:1])
    wide = scale.copy()
    wide[3, 2] = (1 << 45) + 12345                                       # forces the 64-bit scale layout
    hw = q1_gpu.q1_register_weight(bits, wide)
    assert np.array_equal(q1_gpu.q1_apply_resident(hw, x, 200, 8, FRAC), onat.q1_linear(x, bits, wide, FRAC))
    with pytest.raises(ValueError):
        q1_gpu.q1_apply_resident(h64, x[:, :128], 200, 8, FRAC)
    assert q1_gpu.q1_apply_resident(10 ** 6, x, 200, 8, FRAC) is None      # unknown handle: rc 1
    with pytest.raises(ValueError):
        q1_gpu.q1_register_weight(bits, scale, gpu_coalesced=True)          # layouts want int32 scales
    with pytest.raises(TypeError):
        q1_gpu.q1_register_weight(bits, scale.astype(np.float32))


def test_digit_envelope_entry():
    bits, scale, x = _case(21, 32, 2, 2, 20)
    want = onat.q1_linear(x, bits, scale, FRAC)
    assert np.array_equal(q1_gpu.q1_apply_dp4a_gpu(x, bits, scale, FRAC), want)          # picks L = 4
    assert np.array_equal(q1_gpu.q1_apply_dp4a_gpu(x, bits, scale, FRAC, L=-4), want)
    big = x.copy()
    big[1, 5] = 1 << 40
    assert np.array_equal(q1_gpu.q1_apply_dp4a_gpu(big, bits, scale, FRAC), onat.q1_linear(big, bits, scale, FRAC))
    with pytest.raises(ValueError):
        q1_gpu.q1_apply_dp4a_gpu(big, bits, scale, FRAC, L=4)
    lib = q1_gpu.load_library()
    out = np.empty((2, 32), np.int64)
    s64 = np.ascontiguousarray(scale, np.int64)
    rc = lib.bonsai_q1_linear_dp4a_gpu(big.ctypes.data, bits.ctypes.data, s64.ctypes.data, 2, 32, 2, FRAC, 4, out.ctypes.data)
    assert rc == 4                                                                       # the device range guard
    assert lib.bonsai_gpu_last_error_code() == 4
    assert lib.bonsai_q1_linear_dp4a_gpu(big.ctypes.data, bits.ctypes.data, s64.ctypes.data, 2, 32, 2, FRAC, 9, out.ctypes.data) == 1
    assert lib.bonsai_q1_linear_gpu(big.ctypes.data, bits.ctypes.data, s64.ctypes.data, 0, 32, 2, FRAC, out.ctypes.data) == 1


def test_device_entry_and_linearity_at_model_width():
    """d = 4096 -> ffn 12288 of the 8B shape: device entry against the oracle on one token, then a
    size-independent property on a batch: W(x + y) == Wx + Wy fails, because each block floors, but
    W applied to rows one at a time must equal W applied to the batch."""
    import torch

    rng = np.random.default_rng(3)
    bits, scale = o.synth_q1(rng, 12288, 32)
    h = q1_gpu.q1_register_weight(bits, scale.astype(np.int32))
    x = o.to_fixed(rng.standard_normal((40, 4096)), FRAC)
    xd = torch.from_numpy(x).cuda()
    y = q1_gpu.apply_dev(h, xd, FRAC).cpu().numpy()
    assert np.array_equal(y[:2], onat.q1_linear(x[:2], bits, scale, FRAC))
    for t in (0, 17, 39):
        assert np.array_equal(q1_gpu.apply_dev(h, xd[t:t + 1], FRAC).cpu().numpy()[0], y[t])


def test_rmsnorm_entry():
    rng = np.random.default_rng(8)
    x = o.to_fixed(rng.standard_normal((5, 4096)) * 3, FRAC)
    gain = o.to_fixed(1 + rng.standard_normal(4096) * 0.1, FRAC)
    assert np.array_equal(q1_gpu.rmsnorm_gpu(x, FRAC, 1, gain), o.rmsnorm_fixed(x, FRAC, 1, gain))
    assert np.array_equal(q1_gpu.rmsnorm_gpu(x, FRAC, 1), o.rmsnorm_fixed(x, FRAC, 1))
    with pytest.raises(ValueError):
        q1_gpu.rmsnorm_gpu(x, FRAC, 1, gain[:7])
