"""Host-side bridge to the Q1_0 entry points, with the reference bridge's function names.

Mirrors bonsai/src/trinote/infer_int/gpu_native.py:188-415 (``q1_apply_gpu``, ``q1_apply_dp4a_gpu``,
``q1_register_weight``, ``q1_apply_resident``, ``q1_free_weights``, ``rmsnorm_gpu``, ``gpu_memory_info``):
same arguments, same exceptions for malformed input, ``None`` when the library declines a call (rc != 0).
One deliberate difference: a missing library or GPU raises ``CudaUnavailableError`` instead of turning every
function into a silent no-op, because nothing behind this module can take over.

Arrays are host NumPy arrays.  Device-resident callers use :func:`apply_dev` with CUDA tensors.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

import numpy as np

from .qk_cuda import _CUDA_LOCK, CudaUnavailableError

# Every symbol include/iie_q1.h declares; the CPU test-suite checks that the library exports all of them.
EXPORTED_SYMBOLS = (
    "bonsai_gpu_abi_version", "bonsai_gpu_last_error_code", "bonsai_gpu_last_error", "bonsai_gpu_available",
    "bonsai_gpu_mem_info", "bonsai_q1_resident_weight_bytes", "bonsai_q1_linear_gpu", "bonsai_q1_linear_dp4a_gpu",
    "bonsai_q1_register_weight", "bonsai_q1_register_weight_i32", "bonsai_q1_register_weight_i32_gpu_layout",
    "bonsai_q1_register_weight_i32_bmma", "bonsai_q1_apply_resident", "bonsai_q1_free_weights", "bonsai_rmsnorm_gpu",
    "iie_q1_apply_dev", "iie_q1_apply_fused_dev", "iie_q1_head_norm_dev", "iie_q1_silu_mul_dev", "iie_q1_embed_dev", "iie_q1_set_stream", "iie_q1_weight_shape", "iie_q1_workspace_generation",
)
from .qk_cuda import CudaContextError      # noqa: E402  (same error type as the MoE bridge)

_L4_LO, _L4_HI = -2155905152, 2139062143      # balanced base-256 range of four digits (gpu_native.py:223)


def lib_path() -> Path:
    """The build writes one binary under two names: ``libbonsai_q1_gpu.so`` is what the reference's Q1 bridge
    looks for; this module opens ``libnmc_qk_cuda.so`` so that it shares one library instance (launch counter,
    mutex) with :mod:`integer_inference_engine_b200.qk_cuda`."""
    return Path(__file__).resolve().parent / "lib" / "libnmc_qk_cuda.so"


def reference_lib_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libbonsai_q1_gpu.so"


@lru_cache(maxsize=1)
def load_library():
    """``ctypes.CDLL`` of the in-tree library with argument types set; raises if it is not built.
    Loading needs no GPU."""
    p = lib_path()
    if not p.exists():
        raise CudaUnavailableError(f"{p} is not built (python -m integer_inference_engine_b200.build)")
    lib = ctypes.CDLL(str(p))
    missing = [s for s in EXPORTED_SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise CudaUnavailableError(f"{p} lacks symbols {missing}")
    c_int, i64, u64, vp = ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_void_p
    sig = {
        "bonsai_gpu_abi_version": ([], c_int), "bonsai_gpu_last_error_code": ([], c_int),
        "bonsai_gpu_last_error": ([], ctypes.c_char_p), "bonsai_gpu_available": ([], c_int),
        "bonsai_gpu_mem_info": ([vp, vp], c_int), "bonsai_q1_resident_weight_bytes": ([], u64),
        "bonsai_q1_linear_gpu": ([vp, vp, vp, i64, i64, i64, i64, vp], c_int),
        "bonsai_q1_linear_dp4a_gpu": ([vp, vp, vp, i64, i64, i64, i64, c_int, vp], c_int),
        "bonsai_q1_register_weight": ([vp, vp, i64, i64], i64),
        "bonsai_q1_register_weight_i32": ([vp, vp, i64, i64], i64),
        "bonsai_q1_register_weight_i32_gpu_layout": ([vp, vp, i64, i64], i64),
        "bonsai_q1_register_weight_i32_bmma": ([vp, vp, i64, i64], i64),
        "bonsai_q1_apply_resident": ([i64, vp, i64, i64, vp], c_int), "bonsai_q1_free_weights": ([], None),
        "bonsai_rmsnorm_gpu": ([vp, i64, i64, i64, i64, vp, vp], c_int),
        "iie_q1_apply_dev": ([i64, vp, i64, i64, vp, vp], c_int),
        "iie_q1_apply_fused_dev": ([i64, c_int, vp, vp, i64, vp, i64, i64, vp, vp, vp], c_int),
        "iie_q1_head_norm_dev": ([vp, i64, i64, i64, vp, vp, i64, vp, vp], c_int),
        "iie_q1_silu_mul_dev": ([vp, vp, i64, i64, vp, vp], c_int),
        "iie_q1_embed_dev": ([i64, vp, i64, vp, vp], c_int),
        "iie_q1_set_stream": ([c_int], None), "iie_q1_workspace_generation": ([], ctypes.c_uint64),
        "iie_q1_weight_shape": ([i64, ctypes.POINTER(i64), ctypes.POINTER(i64), ctypes.POINTER(c_int)], c_int),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    return lib


def gpu_available() -> bool:
    """True iff the library is built and a usable GPU is present."""
    try:
        return load_library().bonsai_gpu_available() == 0
    except CudaUnavailableError:
        return False


def _lib():
    lib = load_library()
    if lib.bonsai_gpu_available() != 0:
        raise CudaUnavailableError("no usable CUDA device; this package has no CPU path")
    return lib


def _weight_arrays(bits, scale_fp, dtype=np.int64):
    b = np.ascontiguousarray(np.asarray(bits, dtype=np.uint8))
    src = np.asarray(scale_fp)
    if not np.issubdtype(src.dtype, np.integer):
        raise TypeError(f"Q1_0 scale must be an integer dtype, got {src.dtype}")
    s = np.ascontiguousarray(src, dtype=dtype)
    return b, s


def q1_apply_gpu(x_fp, bits, scale_fp, frac: int):
    """Packed Q1_0 linear ``x @ W.T`` with a per-call weight upload (gpu_native.py:193-220)."""
    lib = _lib()
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x_fp, dtype=np.int64)))
    b, s = _weight_arrays(bits, scale_fp)
    out_f, n_blocks = s.shape
    if x.shape[1] != n_blocks * 128:
        raise ValueError(f"Q1_0 contraction mismatch: x has {x.shape[1]}, weight expects {n_blocks * 128}")
    out = np.empty((x.shape[0], out_f), dtype=np.int64)
    with _CUDA_LOCK:
        rc = lib.bonsai_q1_linear_gpu(x.ctypes.data, b.ctypes.data, s.ctypes.data, x.shape[0], int(out_f), int(n_blocks),
                                      int(frac), out.ctypes.data)
    return None if rc != 0 else out


def q1_apply_dp4a_gpu(x_fp, bits, scale_fp, frac: int, L: "int | None" = None):
    """The digit-path entry (gpu_native.py:226-261): ``L`` is the digit count the caller vouches for; an
    explicit ``L=4`` with activations outside the four-digit range raises, as in the reference."""
    lib = _lib()
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x_fp, dtype=np.int64)))
    b, s = _weight_arrays(bits, scale_fp)
    out_f, n_blocks = s.shape
    if x.shape[1] != n_blocks * 128:
        raise ValueError(f"Q1_0 contraction mismatch: x has {x.shape[1]}, weight expects {n_blocks * 128}")
    if L is None:
        mn, mx = (int(x.min()), int(x.max())) if x.size else (0, 0)
        L = 4 if (_L4_LO <= mn and mx <= _L4_HI) else 8
    elif int(L) == 4 and x.size:
        mn, mx = int(x.min()), int(x.max())
        if not (_L4_LO <= mn and mx <= _L4_HI):
            raise ValueError(f"q1_apply_dp4a_gpu: explicit L=4 requires activations in [{_L4_LO}, {_L4_HI}], "
                             f"got [{mn}, {mx}]")
    out = np.empty((x.shape[0], out_f), dtype=np.int64)
    with _CUDA_LOCK:
        rc = lib.bonsai_q1_linear_dp4a_gpu(x.ctypes.data, b.ctypes.data, s.ctypes.data, x.shape[0], int(out_f),
                                           int(n_blocks), int(frac), int(L), out.ctypes.data)
    return None if rc != 0 else out


def residency_available() -> bool:
    return gpu_available()


def q1_register_weight(bits, scale_fp, *, gpu_coalesced: bool = False, gpu_bmma: bool = False):
    """Upload a projection once; returns a handle or ``None`` (gpu_native.py:270-306).  The two layout
    switches are accepted for compatibility and select the same tensor-core layout."""
    lib = _lib()
    src = np.asarray(scale_fp)
    if not np.issubdtype(src.dtype, np.integer):
        raise TypeError(f"Q1_0 scale must be an integer dtype, got {src.dtype}")
    use_i32 = src.dtype.itemsize <= 4
    if gpu_coalesced and gpu_bmma:
        raise ValueError("choose one GPU Q1 runtime layout")
    if (gpu_coalesced or gpu_bmma) and not use_i32:
        raise ValueError("GPU-coalesced Q1 registration currently requires committed int32 scales")
    b, s = _weight_arrays(bits, src, np.int32 if use_i32 else np.int64)
    out_f, n_blocks = s.shape
    if gpu_bmma:
        fn = lib.bonsai_q1_register_weight_i32_bmma
    elif gpu_coalesced:
        fn = lib.bonsai_q1_register_weight_i32_gpu_layout
    else:
        fn = lib.bonsai_q1_register_weight_i32 if use_i32 else lib.bonsai_q1_register_weight
    with _CUDA_LOCK:
        h = fn(b.ctypes.data, s.ctypes.data, int(out_f), int(n_blocks))
    return None if int(h) < 0 else int(h)


def q1_apply_resident(handle: int, x_fp, out_features: int, n_blocks: int, frac: int):
    """Apply a registered weight to fresh host activations (gpu_native.py:364-380)."""
    lib = _lib()
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x_fp, dtype=np.int64)))
    if x.shape[1] != int(n_blocks) * 128:
        raise ValueError(f"Q1_0 contraction mismatch: x has {x.shape[1]}, weight expects {int(n_blocks) * 128}")
    out = np.empty((x.shape[0], int(out_features)), dtype=np.int64)
    with _CUDA_LOCK:
        rc = lib.bonsai_q1_apply_resident(int(handle), x.ctypes.data, x.shape[0], int(frac), out.ctypes.data)
    return None if rc != 0 else out


def q1_free_weights() -> None:
    with _CUDA_LOCK:
        _lib().bonsai_q1_free_weights()


def gpu_memory_info():
    lib = _lib()
    free, total = ctypes.c_uint64(), ctypes.c_uint64()
    if lib.bonsai_gpu_mem_info(ctypes.byref(free), ctypes.byref(total)) != 0:
        return None
    return {"free_bytes": int(free.value), "total_bytes": int(total.value),
            "used_bytes": int(total.value - free.value),
            "resident_weight_bytes": int(lib.bonsai_q1_resident_weight_bytes())}


def rmsnorm_gpu(x_fp, frac: int, eps: int = 1, gain_q=None):
    """Fixed-point RMSNorm of host rows (gpu_native.py:390-415); ``None`` when a row leaves the exact envelope."""
    lib = _lib()
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x_fp, dtype=np.int64)))
    rows, cols = x.shape
    out = np.empty((rows, cols), dtype=np.int64)
    g_ptr, g = 0, None
    if gain_q is not None:
        g = np.ascontiguousarray(np.asarray(gain_q, dtype=np.int64))
        if g.shape[0] != cols:
            raise ValueError(f"RMSNorm gain has {g.shape[0]} elems, expected cols={cols}")
        g_ptr = g.ctypes.data
    with _CUDA_LOCK:
        rc = lib.bonsai_rmsnorm_gpu(x.ctypes.data, rows, cols, int(frac), int(eps), ctypes.c_void_p(g_ptr), out.ctypes.data)
    return None if rc != 0 else out


def apply_dev(handle: int, x, frac: int, out=None):
    """Registered weight times CUDA int64 activations ``[T, n_blocks*128]`` on the current torch stream."""
    import torch

    lib = _lib()
    of, nb, sb = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int()
    if lib.iie_q1_weight_shape(int(handle), ctypes.byref(of), ctypes.byref(nb), ctypes.byref(sb)) != 0:
        raise ValueError(f"unknown Q1_0 weight handle {handle}")
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_cuda or x2.dtype != torch.int64 or not x2.is_contiguous() or x2.shape[1] != nb.value * 128:
        raise ValueError("x must be a contiguous CUDA int64 tensor [T, n_blocks*128]")
    if out is None:
        out = torch.empty((x2.shape[0], of.value), dtype=torch.int64, device=x.device)
    with _CUDA_LOCK:
        rc = lib.iie_q1_apply_dev(int(handle), x2.data_ptr(), x2.shape[0], int(frac), out.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"iie_q1_apply_dev failed with status {rc}")
    return out


def silu_mul_dev(gate, up, frac: int, out=None):
    """((gate * sigmoid(gate)) >> frac) * up >> frac with wrapping products, on CUDA int64 tensors of one shape."""
    import torch

    if out is None:
        out = torch.empty_like(gate)
    rc = _lib().iie_q1_silu_mul_dev(gate.data_ptr(), up.data_ptr(), gate.numel(), int(frac), out.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"iie_q1_silu_mul_dev failed with status {rc}")
    return out


def embed_dev(handle: int, row, out):
    """Row ``row`` (a CUDA int32 cell, or a Python int) of a registered weight as int64 into ``out`` [n_blocks*128]."""
    import torch

    cell = isinstance(row, torch.Tensor)
    rc = _lib().iie_q1_embed_dev(int(handle), row.data_ptr() if cell else None, 0 if cell else int(row), out.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"iie_q1_embed_dev failed with status {rc}")
    return out


def apply_fused_dev(handle: int, x, frac: int, out, *, gain=None, norm: bool = False, up=None, add=None):
    """``out = a W^T (+ add)`` with ``a = x`` (default), ``rmsnorm(x, gain)`` (``norm=True``; ``gain`` a CUDA int64 row or
    None) or the wrapping SwiGLU of ``x`` (gate) and ``up``.  All tensors CUDA int64; ``x`` [T, n_blocks*128] (gate / up may
    be column slices of one [T, ld] tensor); ``add`` may be ``out``."""
    import torch

    mode = 1 if norm else (2 if up is not None else 0)
    T = x.shape[0]
    ld = x.stride(0) if mode == 2 else x.shape[1]
    if mode == 2 and (up.stride(0) != ld or x.stride(1) != 1 or up.stride(1) != 1):
        raise ValueError("gate and up must share one row stride")
    if mode != 2 and not x.is_contiguous():
        raise ValueError("x must be contiguous")
    ptr = lambda t: t.data_ptr() if t is not None else None
    with _CUDA_LOCK:
        rc = _lib().iie_q1_apply_fused_dev(int(handle), mode, x.data_ptr(), ptr(up), int(ld), ptr(gain), int(T), int(frac),
                                           ptr(add), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"iie_q1_apply_fused_dev failed with status {rc}")
    return out


def head_norm_dev(x, rows_a: int, rows_b: int, width: int, gain_a, gain_b, frac: int, out):
    """RMSNorm of ``rows_a + rows_b`` consecutive rows of ``width`` values: the first ``rows_a`` with ``gain_a``, the rest with
    ``gain_b`` (CUDA int64 rows), one launch."""
    import torch

    rc = _lib().iie_q1_head_norm_dev(x.data_ptr(), int(rows_a), int(rows_b), int(width), gain_a.data_ptr(), gain_b.data_ptr(),
                                     int(frac), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"iie_q1_head_norm_dev failed with status {rc}")
    return out


def workspace_generation() -> int:
    """Changes whenever a scratch buffer of the Q1_0 entries is freed; holders of captured graphs compare it."""
    return int(_lib().iie_q1_workspace_generation())


def set_stream_form(on: bool) -> None:
    """Single-token products through the bulk-copy kernel, or (default) the per-lane-load kernel."""
    _lib().iie_q1_set_stream(1 if on else 0)
