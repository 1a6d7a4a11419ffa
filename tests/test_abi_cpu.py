"""CPU suite: the C-ABI library loads without a GPU and exports every symbol include/iie_qk.h
declares; host-side policy helpers behave like the reference bridge's."""
import re
from pathlib import Path

import numpy as np
import pytest

from integer_inference_engine_b200 import build, q1_gpu, qk_cuda

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    build.build()
    return qk_cuda.load_library()


def _declared_symbols():
    text = (ROOT / "include" / "iie_qk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:qk|iie)_[a-z0-9_]+)\s*\(", text)))


def test_header_and_bridge_agree_on_the_symbol_list():
    assert _declared_symbols() == sorted(qk_cuda.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_symbols():
        assert hasattr(lib, name), name
    assert lib.qk_cuda_abi_version() == 5


def test_reference_required_symbols_are_present(lib):
    """The names the reference bridge refuses to load without (north-mini-code/src/nmc/qk_cuda.py:39-72)."""
    required = """qk_cuda_abi_version qk_linear_cuda qk_cuda_available qk_register_weight qk_register_i64
        qk_resident_reserve qk_apply_resident qk_apply_resident_grouped qk_rmsnorm_router qk_attention_bank_create
        qk_attention_bank_import qk_attention_bank_apply qk_attention_bank_moe_configure qk_attention_bank_moe_bind
        qk_attention_bank_moe_begin qk_attention_bank_moe_continue qk_attention_bank_moe_export
        qk_attention_bank_workspace_bytes qk_attention_bank_reset qk_attention_bank_destroy qk_free_all
        qk_resident_count qk_resident_capacity qk_moe_workspace_allocations qk_moe_workspace_bytes
        qk_moe_workspace_release qk_moe_ffn qk_moe_ffn_batched qk_moe_ffn_batched_dp4a qk_profile_reset
        qk_profile_set_enabled qk_profile_snapshot""".split()
    for name in required:
        assert hasattr(lib, name), name


def test_q1_header_bridge_and_library_agree():
    """include/iie_q1.h, the Q1_0 bridge and the library (under the file name the reference's Q1 bridge
    loads) name the same entry points, including the one that bridge treats as mandatory."""
    build.build()
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "iie_q1.h").read_text(), flags=re.S)
    declared = sorted(set(re.findall(r"\b((?:bonsai|iie)_[a-z0-9_]+)\s*\(", text)))
    assert declared == sorted(q1_gpu.EXPORTED_SYMBOLS)
    import ctypes
    lib = q1_gpu.load_library()
    ref_named = ctypes.CDLL(str(q1_gpu.reference_lib_path()))
    for name in declared:
        assert hasattr(lib, name) and hasattr(ref_named, name), name
    assert "bonsai_q1_linear_gpu" in declared and lib.bonsai_gpu_abi_version() == 3
    if not q1_gpu.gpu_available():
        with pytest.raises(q1_gpu.CudaUnavailableError):
            q1_gpu.q1_apply_gpu(np.zeros((1, 128), np.int64), np.zeros((1, 1, 16), np.uint8), np.ones((1, 1), np.int64), 16)


def test_limb_policy_matches_the_capacity_rule():
    """Closed form, the 32640..32767 band two digits cannot hold, and the eight-digit ceiling
    (reference test north-mini-code/tests/test_dp4a_limbs.py:34-79)."""
    for L in range(1, 9):
        cap = qk_cuda._balanced_capacity(L)
        assert cap == sum(127 * 256 ** i for i in range(L))
        assert qk_cuda.limbs_needed(cap) == L
        if L < 8:
            assert qk_cuda.limbs_needed(cap + 1) == L + 1
    for v in range(32640, 32768):
        assert qk_cuda.limbs_needed(v) == 3
    with pytest.raises(OverflowError):
        qk_cuda.limbs_needed(qk_cuda._balanced_capacity(8) + 1)
    x = np.array([qk_cuda._balanced_capacity(8) + 1], dtype=np.int64)
    assert qk_cuda._dp4a_limb_count(x) is None
    with pytest.raises(ValueError):
        qk_cuda._dp4a_limb_count(np.array([1 << 20], dtype=np.int64), 2)


def test_short_weight_buffer_is_refused():
    with pytest.raises(ValueError):
        qk_cuda._require_weight_bytes(b"\0" * 100, 1, 1, qk_cuda.Q4_K)
    with pytest.raises(ValueError):
        qk_cuda._require_weight_bytes(b"\0" * 144, 1, 1, 7)
    assert qk_cuda._require_weight_bytes(b"\0" * 210, 1, 1, qk_cuda.Q6_K) == 210


def test_compute_entries_fail_loudly_without_a_gpu():
    """There is no CPU path behind the bridge."""
    if qk_cuda.available():
        pytest.skip("a GPU is present")
    with pytest.raises(qk_cuda.CudaUnavailableError):
        qk_cuda.qk_linear(b"\0" * 144, np.zeros((1, 256), np.int64), 1, 1, 24, qk_cuda.Q4_K)
    with pytest.raises(qk_cuda.CudaUnavailableError):
        qk_cuda.register_weight(b"\0" * 144, 1, 1, qk_cuda.Q4_K)
