"""Host-side bridge to the Q1_0 entry points of include/iie_q1.h.

The host-array functions carry the names and arguments of the reference's bridge (bonsai/src/trinote/infer_int/
gpu_native.py:188-415: ``q1_apply_gpu``, ``q1_apply_dp4a_gpu``, ``q1_register_weight``, ``q1_apply_resident``,
``q1_free_weights``, ``rmsnorm_gpu``, ``gpu_memory_info``) so its callers can switch modules: malformed input raises,
``None`` means the library declined the call.  Their bodies are this repository's own (two coercion helpers and one
locked call helper).  One deliberate difference: a missing library or GPU raises ``CudaUnavailableError`` instead of
turning every function into a silent no-op, because nothing behind this module can take over.

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
    "bonsai_buf_upload_i64", "bonsai_attention_prefill_gpu", "bonsai_attention_decode_batched_gpu", "bonsai_prefill_forward_gpu",
    "bonsai_decode_ctx_create", "bonsai_decode_ctx_seed_seq", "bonsai_decode_step", "bonsai_decode_ctx_free",
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
        "bonsai_buf_upload_i64": ([vp, i64], i64),
        "bonsai_attention_prefill_gpu": ([vp, vp, vp] + [i64] * 8 + [vp], c_int),
        "bonsai_attention_decode_batched_gpu": ([vp] * 4 + [i64] * 7 + [vp], c_int),
        "bonsai_prefill_forward_gpu": ([vp] + [i64] * 10 + [vp] * 11 + [i64] * 4 + [vp] * 3, c_int),
        "bonsai_decode_ctx_create": ([i64] * 12 + [vp] * 11 + [i64] * 4, i64),
        "bonsai_decode_ctx_seed_seq": ([i64, i64, vp, vp, i64], c_int),
        "bonsai_decode_step": ([i64, vp, vp, vp], c_int), "bonsai_decode_ctx_free": ([i64], None),
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


def _activation(x_fp, n_blocks: int) -> np.ndarray:
    """Host activations as a C-contiguous int64 matrix whose width is the weight's contraction length."""
    x = np.asarray(x_fp, dtype=np.int64)
    x = np.ascontiguousarray(x.reshape(1, -1) if x.ndim < 2 else x)
    if x.shape[1] != int(n_blocks) * 128:
        raise ValueError(f"the activation is {x.shape[1]} wide, the weight contracts over {int(n_blocks) * 128}")
    return x


def _packed_weight(bits, scale_fp, scale_dtype=np.int64):
    """(sign bytes [out_f, n_blocks, 16] uint8, scales [out_f, n_blocks] of ``scale_dtype``), both C-contiguous.
    Scales are committed fixed-point integers: a floating array here is a caller bug, not something to round."""
    scales = np.asarray(scale_fp)
    if scales.dtype.kind not in "iu":
        raise TypeError(f"Q1_0 scales are integers at 2**frac; got dtype {scales.dtype}")
    return np.ascontiguousarray(bits, dtype=np.uint8), np.ascontiguousarray(scales, dtype=scale_dtype)


def _fits_four_digits(x: np.ndarray) -> bool:
    return x.size == 0 or (_L4_LO <= int(x.min()) and int(x.max()) <= _L4_HI)


def _call(name: str, *args) -> int:
    fn = getattr(_lib(), name)
    with _CUDA_LOCK:
        result = fn(*args)
    return 0 if result is None else int(result)


def q1_apply_gpu(x_fp, bits, scale_fp, frac: int):
    """``x @ W.T`` for a packed Q1_0 weight that travels with the call (reference name: gpu_native.py q1_apply_gpu).
    ``None`` when the library declines."""
    b, s = _packed_weight(bits, scale_fp)
    x = _activation(x_fp, s.shape[1])
    y = np.empty((x.shape[0], s.shape[0]), np.int64)
    rc = _call("bonsai_q1_linear_gpu", x.ctypes.data, b.ctypes.data, s.ctypes.data, x.shape[0], s.shape[0], s.shape[1], int(frac),
               y.ctypes.data)
    return y if rc == 0 else None


def q1_apply_dp4a_gpu(x_fp, bits, scale_fp, frac: int, L: "int | None" = None):
    """The entry that takes a digit count ``L`` (reference name: q1_apply_dp4a_gpu).  Without ``L`` the count follows the
    activations (four digits when they fit, else eight); ``L=4`` for activations that need more is refused here, before
    the call, because the native side would have to trust it."""
    b, s = _packed_weight(bits, scale_fp)
    x = _activation(x_fp, s.shape[1])
    if L is None:
        L = 4 if _fits_four_digits(x) else 8
    elif int(L) == 4 and not _fits_four_digits(x):
        raise ValueError(f"L=4 promises activations inside [{_L4_LO}, {_L4_HI}]; these span [{int(x.min())}, {int(x.max())}]")
    y = np.empty((x.shape[0], s.shape[0]), np.int64)
    rc = _call("bonsai_q1_linear_dp4a_gpu", x.ctypes.data, b.ctypes.data, s.ctypes.data, x.shape[0], s.shape[0], s.shape[1],
               int(frac), int(L), y.ctypes.data)
    return y if rc == 0 else None


def residency_available() -> bool:
    return gpu_available()


def q1_register_weight(bits, scale_fp, *, gpu_coalesced: bool = False, gpu_bmma: bool = False):
    """Commit a projection to the device once; its handle, or ``None`` when the library declines.  Scales of at most 32
    bits are kept as int32.  ``gpu_coalesced`` / ``gpu_bmma`` are the reference's layout switches: they exist so that its
    callers need no change and both select the one tensor-core layout this library has."""
    narrow = np.asarray(scale_fp).dtype.itemsize <= 4
    if gpu_coalesced and gpu_bmma:
        raise ValueError("gpu_coalesced and gpu_bmma exclude each other")
    if (gpu_coalesced or gpu_bmma) and not narrow:
        raise ValueError("the layout switches are defined for int32 scales only")
    b, s = _packed_weight(bits, scale_fp, np.int32 if narrow else np.int64)
    entry = ("bonsai_q1_register_weight_i32_bmma" if gpu_bmma else "bonsai_q1_register_weight_i32_gpu_layout" if gpu_coalesced
             else "bonsai_q1_register_weight_i32" if narrow else "bonsai_q1_register_weight")
    handle = _call(entry, b.ctypes.data, s.ctypes.data, s.shape[0], s.shape[1])
    return handle if handle >= 0 else None


def q1_apply_resident(handle: int, x_fp, out_features: int, n_blocks: int, frac: int):
    """Fresh host activations through a registered weight; ``None`` when the library declines."""
    x = _activation(x_fp, n_blocks)
    y = np.empty((x.shape[0], int(out_features)), np.int64)
    rc = _call("bonsai_q1_apply_resident", int(handle), x.ctypes.data, x.shape[0], int(frac), y.ctypes.data)
    return y if rc == 0 else None


def q1_free_weights() -> None:
    _call("bonsai_q1_free_weights")


def gpu_memory_info():
    """Free / total / used device bytes and the bytes registered weights hold, or ``None`` when the query fails."""
    lib = _lib()
    free, total = ctypes.c_uint64(), ctypes.c_uint64()
    if lib.bonsai_gpu_mem_info(ctypes.byref(free), ctypes.byref(total)) != 0:
        return None
    return {"free_bytes": free.value, "total_bytes": total.value, "used_bytes": total.value - free.value,
            "resident_weight_bytes": int(lib.bonsai_q1_resident_weight_bytes())}


def rmsnorm_gpu(x_fp, frac: int, eps: int = 1, gain_q=None):
    """Fixed-point RMSNorm of host rows with an optional gain row; ``None`` when a row leaves the exact envelope."""
    x = np.asarray(x_fp, dtype=np.int64)
    x = np.ascontiguousarray(x.reshape(1, -1) if x.ndim < 2 else x)
    gain = None
    if gain_q is not None:
        gain = np.ascontiguousarray(gain_q, dtype=np.int64).reshape(-1)
        if gain.size != x.shape[1]:
            raise ValueError(f"a gain of {gain.size} values cannot scale rows of {x.shape[1]}")
    y = np.empty_like(x)
    rc = _call("bonsai_rmsnorm_gpu", x.ctypes.data, x.shape[0], x.shape[1], int(frac), int(eps),
               ctypes.c_void_p(gain.ctypes.data if gain is not None else 0), y.ctypes.data)
    return y if rc == 0 else None


# ---- whole-model entries (names and results of bonsai/src/trinote/infer_int/gpu_native.py:418-595) -------------------
def monolith_available() -> bool:
    return gpu_available()


def _i64(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int64))


def buf_upload_i64(arr) -> "int | None":
    """Upload an int64 array once (gains, rope tables); a buffer handle, or ``None`` when the upload failed."""
    flat = _i64(arr).ravel()
    h = int(_call("bonsai_buf_upload_i64", flat.ctypes.data, flat.size))
    return None if h < 0 else h


def attention_prefill_gpu(q_fp, k_fp, v_fp, start: int, frac: int, inv_sqrt_fp: int):
    """Causal attention of M new tokens: q (H, M, hd) after head norm and rotation, k / v (Hkv, L, hd) with L = start + M.
    (H, M, hd) int64, or ``None`` when a value left the exact envelope (the caller's host path decides then)."""
    q, k, v = _i64(q_fp), _i64(k_fp), _i64(v_fp)
    if q.ndim != 3 or k.ndim != 3 or k.shape != v.shape or k.shape[2] != q.shape[2] or k.shape[1] != int(start) + q.shape[1]:
        raise ValueError(f"q {q.shape}, k {k.shape}, v {v.shape} do not describe {q.shape[1] if q.ndim == 3 else '?'} tokens after {start}")
    out = np.empty_like(q)
    rc = _call("bonsai_attention_prefill_gpu", q.ctypes.data, k.ctypes.data, v.ctypes.data, q.shape[0], k.shape[0], q.shape[2],
               q.shape[1], k.shape[1], int(start), int(frac), int(inv_sqrt_fp), out.ctypes.data)
    return out if rc == 0 else None


def attention_decode_batched_gpu(q_fp, Kc, Vc, lengths, frac: int, inv_sqrt_fp: int):
    """One new token of each of B sequences: q (B, H, hd), padded caches (B, Hkv, cap, hd), valid lengths (B,).
    (B, H, hd) int64 or ``None``."""
    q, K, V, n = _i64(q_fp), _i64(Kc), _i64(Vc), _i64(lengths)
    if q.ndim != 3 or K.ndim != 4 or K.shape != V.shape or K.shape[0] != q.shape[0] or K.shape[3] != q.shape[2] or n.shape != (q.shape[0],):
        raise ValueError(f"q {q.shape}, caches {K.shape} / {V.shape}, lengths {n.shape} do not belong together")
    out = np.empty_like(q)
    rc = _call("bonsai_attention_decode_batched_gpu", q.ctypes.data, K.ctypes.data, V.ctypes.data, n.ctypes.data, q.shape[0], q.shape[1],
               K.shape[1], q.shape[2], K.shape[2], int(frac), int(inv_sqrt_fp), out.ctypes.data)
    return out if rc == 0 else None


_WEIGHT_LISTS, _GAIN_LISTS = ("wq", "wk", "wv", "wo", "w1", "wu", "w2"), ("n1g", "n2g", "qng", "kng")


def _handle_lists(w: dict, g: dict, n_layers: int):
    lists = [_i64(w[name]) for name in _WEIGHT_LISTS] + [_i64(g[name]) for name in _GAIN_LISTS]
    if any(a.shape != (n_layers,) for a in lists):
        raise ValueError(f"every per-layer handle list must hold {n_layers} handles")
    return lists


def prefill_forward_gpu(x_embed, dims, w: dict, g: dict, frac: int, eps: int, inv_sqrt_fp: int, *, export_kv: bool = False):
    """The whole prefill on the device.  ``x_embed`` (T, d) embedded rows; ``dims`` = (T, d, n_layers, H, Hkv, hd, dff);
    ``w``: per-layer weight-handle lists wq wk wv wo w1 wu w2, the output matrix ``out_head`` and its row count
    ``out_head_vocab``; ``g``: per-layer buffer-handle lists n1g n2g qng kng and the handles ``finalg``, ``cos_h``,
    ``sin_h``.  Returns the last position's logits (vocab,), with ``export_kv`` also K and V (n_layers, Hkv, T, hd);
    ``None`` (or three of them) when a value left the exact envelope."""
    T, d, n_layers, H, Hkv, hd, dff = (int(v) for v in dims)
    x = _i64(x_embed)
    if x.shape != (T, d):
        raise ValueError(f"x_embed is {x.shape}, dims say ({T}, {d})")
    lists = _handle_lists(w, g, n_layers)
    logits = np.empty(int(w["out_head_vocab"]), dtype=np.int64)
    k = np.empty((n_layers, Hkv, T, hd), dtype=np.int64) if export_kv else None
    v = np.empty_like(k) if export_kv else None
    rc = _call("bonsai_prefill_forward_gpu", x.ctypes.data, T, d, n_layers, H, Hkv, hd, dff, int(frac), int(eps), int(inv_sqrt_fp),
               *[a.ctypes.data for a in lists], int(g["finalg"]), int(w["out_head"]), int(g["cos_h"]), int(g["sin_h"]),
               logits.ctypes.data, k.ctypes.data if export_kv else None, v.ctypes.data if export_kv else None)
    if rc != 0:
        return (None, None, None) if export_kv else None
    return (logits, k, v) if export_kv else logits


def decode_ctx_create(dims, w: dict, g: dict, frac: int, eps: int, inv_sqrt_fp: int, cap: int) -> "int | None":
    """Device decode context of B sequences with ``cap`` cache rows each; ``dims`` = (B, n_layers, H, Hkv, hd, d, dff, vocab)."""
    B, n_layers, H, Hkv, hd, d, dff, vocab = (int(v) for v in dims)
    lists = _handle_lists(w, g, n_layers)
    h = int(_call("bonsai_decode_ctx_create", B, n_layers, H, Hkv, hd, d, dff, int(cap), vocab, int(frac), int(eps), int(inv_sqrt_fp),
                  *[a.ctypes.data for a in lists], int(g["finalg"]), int(w["out_head"]), int(g["cos_h"]), int(g["sin_h"])))
    return None if h < 0 else h


def decode_ctx_seed_seq(ctx: int, b: int, k_arr, v_arr) -> bool:
    """Copy the prefilled K/V rows (n_layers, Hkv, Lb, hd) of sequence ``b`` into the context."""
    k, v = _i64(k_arr), _i64(v_arr)
    if k.ndim != 4 or k.shape != v.shape:
        raise ValueError(f"K {k.shape} and V {v.shape} must both be (n_layers, Hkv, Lb, hd)")
    return _call("bonsai_decode_ctx_seed_seq", int(ctx), int(b), k.ctypes.data, v.ctypes.data, k.shape[2]) == 0


def decode_step(ctx: int, x_in, pos, vocab: int):
    """One token for every sequence of the context: ``x_in`` (B, d) embedded rows, ``pos`` (B,) positions.  (B, vocab)
    logits, or ``None`` on overflow or failure."""
    x, p = _i64(x_in), _i64(pos)
    out = np.empty((x.shape[0], int(vocab)), dtype=np.int64)
    return out if _call("bonsai_decode_step", int(ctx), x.ctypes.data, p.ctypes.data, out.ctypes.data) == 0 else None


def decode_ctx_free(ctx: int) -> None:
    _call("bonsai_decode_ctx_free", int(ctx))


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
