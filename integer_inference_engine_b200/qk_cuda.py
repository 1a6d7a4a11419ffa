"""Host-side bridge to ``libnmc_qk_cuda.so`` with the reference bridge's function names.

Mirrors north-mini-code/src/nmc/qk_cuda.py (names, argument meaning, ``None`` / exception behaviour)
for the MoE hot path, so a caller of ``nmc.qk_cuda`` can switch modules, and tests written against
the reference bridge read the same here.  One deliberate difference: there is no CPU fallback behind
this module.  If the shared library or a GPU is missing, every compute entry raises
``CudaUnavailableError`` instead of returning ``None`` for a caller to fall back on.

All arrays are host NumPy arrays; the library copies them to the device and back.  Device-resident
(PyTorch) callers use :mod:`integer_inference_engine_b200.device` instead.
"""
from __future__ import annotations

import ctypes
import threading
from functools import lru_cache
from pathlib import Path

import numpy as np

Q4_K, Q6_K = 0, 1
_BLOCK_BYTES = {Q4_K: 144, Q6_K: 210}
_CUDA_ABI_VERSION = 5
_DP4A_SAFE_LIMBS = 4
PROFILE_Q, PROFILE_K, PROFILE_V, PROFILE_O, PROFILE_OTHER = 1, 2, 3, 4, 0
_PROFILE_METRICS = (
    "registration_calls", "registration_ns", "h2d_calls", "h2d_bytes", "h2d_ns", "d2h_calls", "d2h_bytes", "d2h_ns",
    "allocation_calls", "allocation_bytes", "allocation_ns", "free_calls", "native_calls", "resident_apply_calls",
    "grouped_apply_calls", "moe_calls", "moe_batched_calls", "moe_batched_dp4a_calls", "q_projection_calls",
    "q_projection_ns", "k_projection_calls", "k_projection_ns", "v_projection_calls", "v_projection_ns",
    "o_projection_calls", "o_projection_ns", "other_projection_calls", "other_projection_ns",
)
# Every symbol include/iie_qk.h declares; the CPU test-suite checks that the library exports all of them.
EXPORTED_SYMBOLS = (
    "qk_cuda_abi_version", "qk_cuda_available", "qk_linear_cuda", "qk_resident_reserve", "qk_register_weight",
    "qk_register_i64", "qk_resident_count", "qk_resident_capacity", "qk_free_all", "qk_apply_resident",
    "qk_apply_resident_grouped", "qk_apply_resident_q6k_dp4a", "qk_apply_resident_q4k_dp4a", "qk_rmsnorm_router",
    "qk_moe_ffn", "qk_moe_ffn_dp4a", "qk_moe_ffn_batched", "qk_moe_ffn_batched_dp4a", "qk_moe_workspace_allocations",
    "qk_moe_workspace_bytes", "qk_moe_workspace_release", "qk_profile_reset", "qk_profile_set_enabled",
    "qk_profile_snapshot", "qk_attention_bank_create", "qk_attention_bank_reset", "qk_attention_bank_destroy",
    "qk_attention_bank_moe_configure", "qk_attention_bank_moe_bind", "qk_attention_bank_import",
    "qk_attention_bank_apply", "qk_attention_bank_moe_begin", "qk_attention_bank_moe_continue",
    "qk_attention_bank_moe_export", "qk_attention_bank_workspace_bytes", "iie_attn_prefill_dev", 
    "iie_register_weight_dev", "iie_weight_export", "iie_moe_layer_create", "iie_moe_layer_destroy",
    "iie_moe_forward_dev", "iie_apply_dev", "iie_flags_read_clear", "iie_rmsnorm_dev", "iie_profile_stage_mask",
    "iie_launch_count", "iie_prefill_launch_counts", "iie_workspace_generation", "iie_moe_block_host", "iie_moe_block_dev", "iie_set_pdl",
    "iie_apply_dev_static", "iie_set_tc_min_tokens", "iie_route_dev", "iie_moe_experts_dev",
    "iie_attn_decode_dev", "iie_embed_dev", "iie_argmax_dev", "iie_attn_block_dev", "iie_set_attn_fused",
    "iie_decoder_create", "iie_decoder_set_layer", "iie_decoder_step_dev", "iie_decoder_destroy",
)
# The library keeps one registry and one set of workspaces per process and ctypes releases the GIL:
# serialise callers here as the reference bridge does (qk_cuda.py:35-38).
_CUDA_LOCK = threading.RLock()


class CudaUnavailableError(RuntimeError):
    """The CUDA library is not built or no GPU is usable; there is no fallback path."""


class CudaRegistrationError(RuntimeError):
    """A resident weight could not be committed to device memory."""


class CudaContextError(RuntimeError):
    """A resident call failed validation, allocation, or an exact-envelope guard."""


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libnmc_qk_cuda.so"


@lru_cache(maxsize=1)
def load_library():
    """``ctypes.CDLL`` of the in-tree library with argument types set; raises if it is not built.
    Loading needs no GPU (the CPU test-suite checks the exported symbols this way)."""
    p = lib_path()
    if not p.exists():
        raise CudaUnavailableError(f"{p} is not built (python -m integer_inference_engine_b200.build)")
    lib = ctypes.CDLL(str(p))
    missing = [s for s in EXPORTED_SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise CudaUnavailableError(f"{p} lacks symbols {missing}")
    c_int, i64, u64, vp = ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_void_p
    P64, P32 = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int)
    sig = {
        "qk_cuda_abi_version": ([], c_int), "qk_cuda_available": ([], c_int),
        "qk_linear_cuda": ([vp, vp, i64, i64, i64, c_int, c_int, vp], c_int),
        "qk_resident_reserve": ([i64], c_int), "qk_register_weight": ([vp, i64, i64, c_int], i64),
        "qk_register_i64": ([vp, i64, i64], i64), "qk_resident_count": ([], i64), "qk_resident_capacity": ([], i64),
        "qk_free_all": ([], None), "qk_apply_resident": ([i64, vp, i64, c_int, vp], c_int),
        "qk_apply_resident_grouped": ([P64, P32, c_int, vp, i64, c_int, i64, vp], c_int),
        "qk_apply_resident_q6k_dp4a": ([i64, vp, i64, c_int, c_int, vp], c_int),
        "qk_apply_resident_q4k_dp4a": ([i64, vp, i64, c_int, c_int, vp], c_int),
        "qk_rmsnorm_router": ([i64, i64, vp, i64, c_int, c_int, u64, c_int, i64, i64, vp, vp, vp], c_int),
        "qk_moe_ffn": ([P64, P64, P64, c_int, vp, vp, i64, i64, c_int, c_int, vp], c_int),
        "qk_moe_ffn_dp4a": ([P64, P64, P64, c_int, vp, vp, i64, i64, c_int, c_int, vp], c_int),
        "qk_moe_ffn_batched": ([P64, P64, P64, c_int, c_int, vp, vp, i64, i64, c_int, c_int, vp], c_int),
        "qk_moe_ffn_batched_dp4a": ([P64, P64, P64, c_int, c_int, vp, vp, i64, i64, c_int, c_int, vp], c_int),
        "qk_moe_workspace_allocations": ([], i64), "qk_moe_workspace_bytes": ([], u64),
        "qk_moe_workspace_release": ([], None), "qk_profile_reset": ([], None),
        "qk_profile_set_enabled": ([c_int], None),
        "qk_profile_snapshot": ([ctypes.POINTER(ctypes.c_uint64), c_int], c_int),
        "qk_attention_bank_create": ([c_int, i64, i64, c_int, c_int, c_int, c_int, vp, vp], i64),
        "qk_attention_bank_reset": ([i64], c_int), "qk_attention_bank_destroy": ([i64], None),
        "qk_attention_bank_import": ([i64, c_int, vp, vp, i64], c_int),
        "qk_attention_bank_apply": ([i64, c_int, i64, i64, i64, i64, vp, c_int, c_int, c_int, i64, i64, vp], c_int),
        "qk_attention_bank_workspace_bytes": ([i64], u64),
        "iie_register_weight_dev": ([vp, i64, i64, c_int], i64), "iie_weight_export": ([i64, vp], c_int),
        "iie_moe_layer_create": ([i64, P64, P64, P64, c_int, c_int, i64, i64], i64),
        "iie_moe_layer_destroy": ([i64], None),
        "iie_moe_forward_dev": ([i64, vp, i64, c_int, c_int, c_int, vp, vp, vp, vp], c_int),
        "iie_apply_dev": ([i64, vp, i64, c_int, vp, vp], c_int), "iie_flags_read_clear": ([vp], c_int),
        "iie_apply_dev_static": ([i64, vp, i64, c_int, vp, vp], c_int),
        "iie_rmsnorm_dev": ([i64, vp, i64, i64, c_int, u64, vp, vp], c_int),
        "iie_profile_stage_mask": ([c_int], None), "iie_launch_count": ([], u64), "iie_set_pdl": ([c_int], None),
        "iie_set_tc_min_tokens": ([i64], None), 
        "iie_attn_decode_dev": ([vp, vp, vp, vp, vp, i64, vp, i64, vp, vp, c_int, c_int, c_int, c_int, i64, c_int, i64, vp, vp], c_int),
        "iie_attn_prefill_dev": ([vp, vp, vp, vp, vp, i64, i64, i64, vp, vp, c_int, c_int, c_int, c_int, i64, c_int, i64, vp, vp], c_int),
        "iie_decoder_create": ([c_int, c_int, c_int, c_int, i64, i64, c_int, c_int, u64, i64, vp, vp], i64),
        "iie_decoder_set_layer": ([i64, c_int, i64, i64, i64, i64, vp, vp, c_int], c_int),
        "iie_decoder_step_dev": ([i64, vp, i64, vp, vp, vp, vp], c_int), "iie_decoder_destroy": ([i64], None),
        "iie_prefill_launch_counts": ([ctypes.POINTER(ctypes.c_uint64), c_int], c_int), "iie_workspace_generation": ([], u64),
        "iie_attn_block_dev": ([i64, i64, vp, vp, vp, i64, vp, i64, vp, vp, c_int, c_int, c_int, c_int, i64, c_int, c_int, i64, vp], c_int),
        "iie_embed_dev": ([i64, vp, i64, c_int, vp, vp], c_int), "iie_set_attn_fused": ([c_int], None), "iie_argmax_dev": ([vp, i64, vp, vp], c_int),
        "iie_route_dev": ([i64, c_int, vp, i64, c_int, c_int, vp, vp, vp], c_int),
        "iie_moe_experts_dev": ([i64, vp, i64, vp, vp, c_int, c_int, c_int, c_int, c_int, vp, vp], c_int),
        "iie_moe_block_host": ([i64, i64, vp, i64, c_int, c_int, u64, vp, vp, vp], c_int),
        "iie_moe_block_dev": ([i64, i64, vp, i64, c_int, c_int, u64, vp, vp, vp, vp], c_int),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    if int(lib.qk_cuda_abi_version()) != _CUDA_ABI_VERSION:
        raise CudaUnavailableError("library reports a different ABI version")
    return lib


@lru_cache(maxsize=1)
def _gpu_ok() -> bool:
    with _CUDA_LOCK:
        return load_library().qk_cuda_available() == 0


def available() -> bool:
    """True when the library is built and a GPU is usable."""
    try:
        return _gpu_ok()
    except CudaUnavailableError:
        return False


def _lib():
    lib = load_library()
    if not _gpu_ok():
        raise CudaUnavailableError("no usable CUDA device; this package has no CPU path")
    return lib


def _require_weight_bytes(weight_raw, out_f: int, n_blocks: int, qtype: int) -> int:
    """The kernel reads out_f*n_blocks*block_bytes bytes: refuse a shorter buffer
    (north-mini-code/src/nmc/qk_native.py:19-31)."""
    bs = _BLOCK_BYTES.get(int(qtype))
    if bs is None:
        raise ValueError(f"unknown qtype {qtype} (expected Q4_K={Q4_K} or Q6_K={Q6_K})")
    out_f, n_blocks = int(out_f), int(n_blocks)
    if out_f <= 0 or n_blocks <= 0:
        raise ValueError(f"out_f and n_blocks must be positive, got out_f={out_f}, n_blocks={n_blocks}")
    need = out_f * n_blocks * bs
    if len(weight_raw) < need:
        raise ValueError(f"weight buffer too short: {len(weight_raw)} bytes < required {need}")
    return need


def _bytes_ptr(raw):
    buf = np.frombuffer(raw, np.uint8) if not isinstance(raw, np.ndarray) else np.ascontiguousarray(raw).view(np.uint8)
    return buf, buf.ctypes.data


def _x2d(x_int) -> np.ndarray:
    return np.ascontiguousarray(np.atleast_2d(np.asarray(x_int, dtype=np.int64)))


# ------------------------------------------------------------------------------------- linear / residency ---
def qk_linear(weight_raw, x_int, out_f: int, n_blocks: int, fw: int, qtype: int):
    """y[t,o] = (sum_i W[o,i]*x[t,i]) >> fw from raw Q4_K/Q6_K bytes; x [T,in_f] int64 -> [T,out_f] int64.
    ``None`` on a native failure (qk_cuda.py:230-244)."""
    lib = _lib()
    x = _x2d(x_int)
    assert x.shape[1] == n_blocks * 256, (x.shape, n_blocks)
    _require_weight_bytes(weight_raw, out_f, n_blocks, qtype)
    keep, wp = _bytes_ptr(weight_raw)
    out = np.empty((x.shape[0], out_f), np.int64)
    with _CUDA_LOCK:
        rc = lib.qk_linear_cuda(wp, x.ctypes.data, x.shape[0], out_f, n_blocks, int(fw), int(qtype), out.ctypes.data)
    return None if rc != 0 else out


def resident_available() -> bool:
    return available()


def register_weight(weight_raw, out_f: int, n_blocks: int, qtype: int) -> int:
    """Upload a weight tensor once; returns its handle, raises on failure (qk_cuda.py:252-271)."""
    lib = _lib()
    _require_weight_bytes(weight_raw, out_f, n_blocks, qtype)
    keep, wp = _bytes_ptr(weight_raw)
    with _CUDA_LOCK:
        h = lib.qk_register_weight(wp, out_f, n_blocks, qtype)
    if h < 0:
        raise CudaRegistrationError(f"registration failed for shape [{out_f}, {n_blocks * 256}] (qtype={qtype})")
    return int(h)


def register_i64(matrix) -> int:
    """Upload a dense int64 matrix (a vector becomes one row) for RMSNorm gains and dense routers
    (qk_cuda.py:280-304)."""
    lib = _lib()
    value = np.asarray(matrix, dtype=np.int64)
    if value.ndim == 1:
        value = value.reshape(1, -1)
    if value.ndim != 2 or value.shape[0] <= 0 or value.shape[1] <= 0:
        raise ValueError("resident int64 registration requires a non-empty vector or 2-D matrix")
    value = np.ascontiguousarray(value)
    with _CUDA_LOCK:
        h = int(lib.qk_register_i64(value.ctypes.data, value.shape[0], value.shape[1]))
    if h < 0:
        raise CudaRegistrationError(f"int64 registration failed for shape {value.shape}")
    return h


def reserve_resident_capacity(count: int) -> bool:
    with _CUDA_LOCK:
        return _lib().qk_resident_reserve(int(count)) == 0


def resident_count() -> int:
    with _CUDA_LOCK:
        return int(_lib().qk_resident_count())


def resident_capacity() -> int:
    with _CUDA_LOCK:
        return int(_lib().qk_resident_capacity())


def free_all() -> None:
    with _CUDA_LOCK:
        _lib().qk_free_all()


def apply_resident(handle: int, x_int, out_f: int, fw: int):
    """Apply a resident weight; ``None`` for a bad handle or native failure (qk_cuda.py:387-397)."""
    lib = _lib()
    x = _x2d(x_int)
    out = np.empty((x.shape[0], out_f), np.int64)
    with _CUDA_LOCK:
        rc = lib.qk_apply_resident(int(handle), x.ctypes.data, x.shape[0], int(fw), out.ctypes.data)
    return None if rc != 0 else out


def grouped_available() -> bool:
    return available()


def apply_resident_grouped(handles, x_int, out_features, fw: int, phase_ids=None):
    """Same input through several resident weights with one upload and one download; results in
    handle order (qk_cuda.py:405-442)."""
    lib = _lib()
    hs = tuple(int(h) for h in handles)
    ofs = tuple(int(n) for n in out_features)
    if not hs or len(hs) != len(ofs) or len(hs) > 16 or any(n <= 0 for n in ofs):
        raise ValueError("grouped resident apply requires 1..16 handles and matching positive output sizes")
    phases = tuple(PROFILE_OTHER for _ in hs) if phase_ids is None else tuple(int(p) for p in phase_ids)
    if len(phases) != len(hs) or any(p not in (0, 1, 2, 3, 4) for p in phases):
        raise ValueError("grouped resident phase_ids must match handles and use known identifiers")
    x = _x2d(x_int)
    rows = int(x.shape[0])
    total = rows * sum(ofs)
    flat = np.empty(total, np.int64)
    harr = (ctypes.c_int64 * len(hs))(*hs)
    parr = (ctypes.c_int * len(hs))(*phases)
    with _CUDA_LOCK:
        rc = lib.qk_apply_resident_grouped(harr, parr, len(hs), x.ctypes.data, rows, int(fw), total, flat.ctypes.data)
    if rc != 0:
        return None
    result, off = [], 0
    for n in ofs:
        result.append(flat[off:off + rows * n].reshape(rows, n))
        off += rows * n
    return tuple(result)


# ------------------------------------------------------------------------------------------- limb policy ---
def _balanced_capacity(L: int) -> int:
    """Largest |x| that L balanced base-256 digits represent: 127*(256^L-1)/255 (qk_cuda.py:973-976)."""
    return 127 * ((256 ** L - 1) // 255)


def limbs_needed(maxabs: int) -> int:
    """Smallest digit count 1..8 covering +-maxabs; OverflowError beyond eight (qk_cuda.py:979-992)."""
    m = int(maxabs)
    L = 1
    while L < 8 and m > _balanced_capacity(L):
        L += 1
    if m > _balanced_capacity(8):
        raise OverflowError(f"|x| max {m} exceeds 8 balanced base-256 digits ({_balanced_capacity(8)})")
    return L


def _activation_absmax(x: np.ndarray) -> int:
    return max(abs(int(x.min())), abs(int(x.max()))) if x.size else 0


def _dp4a_limb_count(x: np.ndarray, requested=None):
    """Digit count for the type-specific applies.  The kernels here always carry eight digits and
    recombine them in 128 bits, so any count up to eight is exact; ``None`` means the activation
    needs a ninth digit and the caller must use :func:`apply_resident` (which then takes the
    128-bit kernel).  An explicit count that is too small or out of range is a caller error."""
    try:
        needed = limbs_needed(_activation_absmax(x))
    except OverflowError:
        if requested is None:
            return None
        raise ValueError("activation is not representable by eight balanced base-256 digits") from None
    if requested is None:
        return needed
    requested = int(requested)
    if not 1 <= requested <= 8:
        raise ValueError(f"limb count must be in [1, 8], got {requested}")
    if requested < needed:
        raise ValueError(f"limb count {requested} is too small; activation requires {needed}")
    return requested


def dp4a_available() -> bool:
    return available()


def apply_resident_dp4a(handle: int, x_int, out_f: int, fw: int, qtype: int, ln=None):
    """Type-checked apply of a resident Q4_K / Q6_K weight, byte-identical to :func:`apply_resident`
    (qk_cuda.py:1029-1050).  ``None`` when the handle has the other type or the activation needs a
    ninth digit."""
    if qtype not in (Q4_K, Q6_K):
        raise ValueError(f"unknown qtype {qtype} (expected Q4_K={Q4_K} or Q6_K={Q6_K})")
    lib = _lib()
    fn = lib.qk_apply_resident_q4k_dp4a if qtype == Q4_K else lib.qk_apply_resident_q6k_dp4a
    x = _x2d(x_int)
    ln = _dp4a_limb_count(x, ln)
    if ln is None:
        return None
    out = np.empty((x.shape[0], out_f), np.int64)
    with _CUDA_LOCK:
        rc = fn(int(handle), x.ctypes.data, x.shape[0], int(fw), int(ln), out.ctypes.data)
    return None if rc != 0 else out


def apply_resident_q6k_dp4a(handle: int, x_int, out_f: int, fw: int, ln=None):
    return apply_resident_dp4a(handle, x_int, out_f, fw, Q6_K, ln)


# ------------------------------------------------------------------------------------- router / MoE block ---
_I128_MAX = (1 << 127) - 1


def _rmsnorm_i128_safe(x: np.ndarray) -> bool:
    """Each row's sum of squares must fit a signed 128-bit integer (qk_cuda.py:310-328)."""
    if x.ndim != 2 or x.shape[1] <= 0:
        return False
    width = int(x.shape[1])
    for row in x:
        maxabs = max(abs(int(row.min())), abs(int(row.max())))
        if maxabs * maxabs * width <= _I128_MAX:
            continue
        total = 0
        for v in row:
            total += int(v) * int(v)
            if total > _I128_MAX:
                return False
    return True


def resident_preprocess_available() -> bool:
    return available()


def rmsnorm_router(gain_handle: int, router_handle: int, x_int, n_used: int, fa: int, fw: int, eps: int = 1):
    """Exact RMSNorm, dense int64 router product, top-k (lowest index on ties) and sigmoid gates.
    Returns (h [T,D], ids [T,K] int32, gates [T,K]) or ``None`` when the activation leaves the exact
    envelope; shape/runtime failures raise (qk_cuda.py:331-372)."""
    lib = _lib()
    x = np.asarray(x_int, dtype=np.int64)
    if x.ndim == 1:
        x = x.reshape(1, -1)
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] <= 0:
        raise ValueError("resident RMSNorm/router requires a non-empty vector or 2-D activation")
    x = np.ascontiguousarray(x)
    n_used, fa, fw, eps = int(n_used), int(fa), int(fw), int(eps)
    if not 0 < n_used <= np.iinfo(np.int32).max:
        raise ValueError("n_used out of range")
    if not 1 <= fa <= 29 or not 0 <= fw <= 62 or not 0 <= eps <= (1 << 64) - 1:
        raise ValueError("fixed-point parameters are outside the native envelope")
    if not _rmsnorm_i128_safe(x):
        return None
    rows = int(x.shape[0])
    h = np.empty_like(x)
    ids = np.empty((rows, n_used), np.int32)
    gates = np.empty((rows, n_used), np.int64)
    with _CUDA_LOCK:
        rc = int(lib.qk_rmsnorm_router(int(gain_handle), int(router_handle), x.ctypes.data, rows, fa, fw, eps, n_used,
                                       h.size, ids.size, h.ctypes.data, ids.ctypes.data, gates.ctypes.data))
    if rc == 3:
        return None
    if rc != 0:
        raise CudaContextError(f"resident RMSNorm/router failed with native status {rc}")
    return h, ids, gates


def moe_ffn_available() -> bool:
    return available()


moe_ffn_dp4a_available = moe_ffn_batched_available = moe_ffn_batched_dp4a_available = moe_ffn_available


def moe_ffn(gate_h, up_h, down_h, h, gates, d_model: int, e_ffn: int, fa: int, fw: int, dp4a: bool = False):
    """Decode MoE expert FFN on one token: out[d_model] = sum_e ((down_e(silu(gate_e h) * up_e h) * g_e) >> fa).
    ``dp4a`` selects the type-specific entry name; both produce identical bytes (qk_cuda.py:1104-1124)."""
    lib = _lib()
    fn = lib.qk_moe_ffn_dp4a if dp4a else lib.qk_moe_ffn
    n_e = len(gate_h)
    if n_e <= 0 or len(up_h) != n_e or len(down_h) != n_e:
        raise ValueError("MoE requires the same positive number of gate, up, and down handles")
    arr = lambda hs: (ctypes.c_int64 * n_e)(*[int(v) for v in hs])
    hh = np.ascontiguousarray(np.asarray(h, np.int64).reshape(-1))
    gg = np.ascontiguousarray(np.asarray(gates, np.int64).reshape(-1))
    if hh.size != d_model or gg.size != n_e:
        raise ValueError(f"MoE expected h.size={d_model} and gates.size={n_e}, got {hh.size} and {gg.size}")
    out = np.empty(int(d_model), np.int64)
    with _CUDA_LOCK:
        rc = fn(arr(gate_h), arr(up_h), arr(down_h), n_e, hh.ctypes.data, gg.ctypes.data, int(d_model), int(e_ffn),
                int(fa), int(fw), out.ctypes.data)
    return None if rc != 0 else out


def moe_ffn_batched(gate_h, up_h, down_h, m: int, k: int, h, gates, d_model: int, e_ffn: int, fa: int, fw: int, *,
                    dp4a: bool = False):
    """Batched MoE over all m*k (token, selected expert) pairs, handles flattened token-major
    (pair = t*k + j); h [m,d_model], gates [m*k] -> [m,d_model] (qk_cuda.py:1073-1101)."""
    lib = _lib()
    P = m * k
    if m <= 0 or k <= 0:
        raise ValueError(f"batched MoE requires positive m and k, got m={m}, k={k}")
    if len(gate_h) != P or len(up_h) != P or len(down_h) != P:
        raise ValueError(f"batched MoE requires exactly m*k={P} handles for each projection")
    arr = lambda hs: (ctypes.c_int64 * P)(*[int(v) for v in hs])
    hh = np.ascontiguousarray(np.asarray(h, np.int64).reshape(-1))
    gg = np.ascontiguousarray(np.asarray(gates, np.int64).reshape(-1))
    if hh.size != m * d_model or gg.size != P:
        raise ValueError(f"batched MoE expected h.size={m * d_model} and gates.size={P}")
    out = np.empty((m, d_model), np.int64)
    with _CUDA_LOCK:
        args = (arr(gate_h), arr(up_h), arr(down_h), int(m), int(k), hh.ctypes.data, gg.ctypes.data, int(d_model),
                int(e_ffn), int(fa), int(fw), out.ctypes.data)
        use_dp4a = bool(dp4a and _dp4a_limb_count(hh) is not None and
                        limbs_needed(_activation_absmax(hh)) <= _DP4A_SAFE_LIMBS)
        rc = lib.qk_moe_ffn_batched_dp4a(*args) if use_dp4a else lib.qk_moe_ffn_batched(*args)
        if use_dp4a and rc == 2:
            rc = lib.qk_moe_ffn_batched(*args)
    return None if rc != 0 else out


def moe_workspace_allocations():
    with _CUDA_LOCK:
        return int(_lib().qk_moe_workspace_allocations())


def moe_workspace_bytes():
    with _CUDA_LOCK:
        return int(_lib().qk_moe_workspace_bytes())


def release_moe_workspace() -> bool:
    with _CUDA_LOCK:
        _lib().qk_moe_workspace_release()
    return True


# ------------------------------------------------------------------------------------------------ profile ---
def profile_reset(*, enabled: bool = True) -> bool:
    """Zero the native counters and switch collection on or off (qk_cuda.py:870-879)."""
    lib = _lib()
    with _CUDA_LOCK:
        lib.qk_profile_set_enabled(0)
        lib.qk_profile_reset()
        lib.qk_profile_set_enabled(int(bool(enabled)))
    return True


def profile_set_enabled(enabled: bool) -> bool:
    with _CUDA_LOCK:
        _lib().qk_profile_set_enabled(1 if enabled else 0)
    return True


def profile_snapshot() -> dict:
    buf = (ctypes.c_uint64 * len(_PROFILE_METRICS))()
    with _CUDA_LOCK:
        n = _lib().qk_profile_snapshot(buf, len(_PROFILE_METRICS))
    if n != len(_PROFILE_METRICS):
        raise CudaContextError("profile snapshot size mismatch")
    return {name: int(buf[i]) for i, name in enumerate(_PROFILE_METRICS)}


def resident_attention_available() -> bool:
    """True when the request-scoped attention bank can be used (qk_cuda.py:471-473 of the reference bridge)."""
    return available()


class ResidentAttentionCache:
    """Request-scoped device K/V bank and exact single-token attention sublayer; names, arguments and error behaviour of
    north-mini-code/src/nmc/qk_cuda.py:476-569.  A prefill's K/V is imported once per layer; every ``apply`` then takes
    one normalised hidden row and returns the projected attention row, appending the new K/V row on the device.  A failed
    call poisons that layer and raises; the caller closes the context instead of retrying."""

    def __init__(self, n_layers: int, max_length: int, d_model: int, n_heads: int, n_kv: int, head_dim: int, fa: int, cos, sin):
        lib = _lib()
        n_layers, max_length, d_model, n_heads, n_kv, head_dim, fa = (int(v) for v in (n_layers, max_length, d_model, n_heads,
                                                                                        n_kv, head_dim, fa))
        q_width = n_heads * head_dim
        if n_layers <= 0 or max_length <= 0 or d_model <= 0 or n_heads <= 0 or n_kv <= 0 or n_heads % n_kv or head_dim <= 0 or \
                head_dim % 2 or not 1 <= fa <= 29 or d_model % 256 or q_width % 256:
            raise ValueError("invalid resident attention dimensions")
        c = np.ascontiguousarray(np.asarray(cos, dtype=np.int64))
        s = np.ascontiguousarray(np.asarray(sin, dtype=np.int64))
        expected = (max_length, head_dim // 2)
        if c.shape != expected or s.shape != expected:
            raise ValueError(f"resident attention RoPE tables must both have shape {expected}")
        with _CUDA_LOCK:
            handle = int(lib.qk_attention_bank_create(n_layers, max_length, d_model, n_heads, n_kv, head_dim, fa,
                                                      c.ctypes.data, s.ctypes.data))
        if handle < 0:
            raise CudaContextError("resident attention context creation failed; check dimensions and VRAM")
        self.handle = handle
        self.n_layers, self.max_length = n_layers, max_length
        self.n_heads, self.n_kv, self.head_dim, self.fa = n_heads, n_kv, head_dim, fa
        self.d_model, self.q_width = d_model, q_width
        self._lengths = [0] * n_layers
        self._closed = False

    def length(self, layer=0):
        return self._lengths[layer]

    def import_layer(self, layer: int, k, v) -> None:
        if self._closed:
            raise CudaContextError("resident attention context is closed")
        layer = int(layer)
        kk = np.ascontiguousarray(np.asarray(k, dtype=np.int64))
        vv = np.ascontiguousarray(np.asarray(v, dtype=np.int64))
        if kk.shape != vv.shape or kk.ndim != 3 or kk.shape[0] != self.n_kv or kk.shape[2] != self.head_dim:
            raise ValueError("resident attention import expects matching [n_kv, length, head_dim] K/V")
        length = int(kk.shape[1])
        if not 0 <= layer < self.n_layers or length > self.max_length:
            raise ValueError("resident attention import exceeds layer or context bounds")
        with _CUDA_LOCK:
            rc = _lib().qk_attention_bank_import(self.handle, layer, kk.ctypes.data, vv.ctypes.data, length)
        if rc != 0:
            raise CudaContextError(f"resident attention K/V import failed for layer {layer}")
        self._lengths[layer] = length

    def apply(self, layer: int, q_handle: int, k_handle: int, v_handle: int, o_handle: int, hidden, fw: int,
              window: "int | None", rope: bool):
        if self._closed:
            raise CudaContextError("resident attention context is closed")
        layer = int(layer)
        if not 0 <= layer < self.n_layers or self._lengths[layer] >= self.max_length:
            raise ValueError("resident attention decode exceeds layer or context bounds")
        x = np.ascontiguousarray(np.asarray(hidden, dtype=np.int64))
        if x.shape != (1, self.d_model):
            raise ValueError(f"resident attention apply expects hidden shape (1, {self.d_model})")
        out = np.empty((1, self.d_model), dtype=np.int64)
        inv_sqrt = int(round((1.0 / self.head_dim ** 0.5) * (1 << self.fa)))
        with _CUDA_LOCK:
            rc = int(_lib().qk_attention_bank_apply(self.handle, layer, int(q_handle), int(k_handle), int(v_handle), int(o_handle),
                                                    x.ctypes.data, int(fw), -1 if window is None else int(window),
                                                    int(bool(rope)), inv_sqrt, out.size, out.ctypes.data))
        if rc != 0:
            detail = "exact overflow guard fired" if rc == 3 else f"native status {rc}"
            raise CudaContextError(f"resident attention apply failed for layer {layer}: {detail}")
        self._lengths[layer] += 1
        return out

    def reset(self) -> None:
        if self._closed:
            raise CudaContextError("resident attention context is closed")
        with _CUDA_LOCK:
            rc = _lib().qk_attention_bank_reset(self.handle)
        if rc != 0:
            raise CudaContextError("resident attention reset failed")
        self._lengths = [0] * self.n_layers

    def workspace_bytes(self) -> int:
        with _CUDA_LOCK:
            return int(_lib().qk_attention_bank_workspace_bytes(self.handle))

    def close(self) -> None:
        if not self._closed:
            with _CUDA_LOCK:
                _lib().qk_attention_bank_destroy(self.handle)
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def moe_block(layer_handle: int, x_int, n_used: int, fa: int, fw: int, gain_handle: int = -1, eps: int = 1):
    """Whole MoE block on host arrays in one native call: ``moe(x)`` or, with a gain handle,
    ``x + moe(rmsnorm(x, gain))``.  Returns (out [T,d], ids [T,k] int32, gates [T,k]) or ``None`` when an
    input leaves the exact envelope.  Additive entry (no counterpart in the reference bridge): it
    replaces the per-layer sequence rmsnorm_router + moe_ffn with one upload and one download."""
    lib = _lib()
    x = _x2d(x_int)
    out = np.empty_like(x)
    ids = np.empty((x.shape[0], int(n_used)), np.int32)
    gates = np.empty((x.shape[0], int(n_used)), np.int64)
    with _CUDA_LOCK:
        rc = lib.iie_moe_block_host(int(layer_handle), int(gain_handle), x.ctypes.data, x.shape[0], int(fa), int(fw),
                                    int(eps), out.ctypes.data, ids.ctypes.data, gates.ctypes.data)
    if rc == 3:
        return None
    if rc != 0:
        raise CudaContextError(f"MoE block failed with native status {rc}")
    return out, ids, gates
