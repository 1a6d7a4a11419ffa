"""Host-side bridge to ``libnmc_qk_cuda.so``: NumPy arrays in, NumPy arrays out, through the C-ABI of include/iie_qk.h.

The public names and their meaning are those of the reference's bridge module (north-mini-code/src/nmc/qk_cuda.py), so
that a caller of ``nmc.qk_cuda`` finds the same calls here: ``register_weight`` / ``apply_resident*`` (qk_cuda.py:230-442),
``rmsnorm_router`` (:331-372), ``moe_ffn`` / ``moe_ffn_batched`` (:1073-1124), the limb policy (:973-1026), the profile
counters (:870-900) and the request-scoped attention bank (:476-569).  How they are written is this repository's own: one
table of C signatures drives both the symbol check and the ctypes set-up, array arguments go through two small coercion
helpers, and every native call goes through :func:`_native`, which takes the process-wide lock.

One deliberate difference from the reference: nothing here falls back to a CPU path.  Without the built library or a
usable GPU every compute entry raises :class:`CudaUnavailableError`; a native status that the reference maps to "use the
host path" is handed to the caller as ``None`` exactly as there, and it is the caller who owns that decision.

Device-resident (PyTorch) callers use :mod:`integer_inference_engine_b200.device` instead; it shares this module's
library instance, lock and error types.
"""
from __future__ import annotations

import ctypes
import threading
from functools import lru_cache
from pathlib import Path

import numpy as np

Q4_K, Q6_K = 0, 1
_BLOCK_BYTES = {Q4_K: 144, Q6_K: 210}
PROFILE_OTHER, PROFILE_Q, PROFILE_K, PROFILE_V, PROFILE_O = 0, 1, 2, 3, 4
# counter order of qk_profile_snapshot (the ABI fixes it)
_PROFILE_METRICS = (
    "registration_calls", "registration_ns", "h2d_calls", "h2d_bytes", "h2d_ns", "d2h_calls", "d2h_bytes", "d2h_ns",
    "allocation_calls", "allocation_bytes", "allocation_ns", "free_calls", "native_calls", "resident_apply_calls",
    "grouped_apply_calls", "moe_calls", "moe_batched_calls", "moe_batched_dp4a_calls", "q_projection_calls",
    "q_projection_ns", "k_projection_calls", "k_projection_ns", "v_projection_calls", "v_projection_ns",
    "o_projection_calls", "o_projection_ns", "other_projection_calls", "other_projection_ns",
)
_MAX_GROUP = 16          # handles one grouped apply may carry (the ABI's limit)
_DIGITS = 8              # balanced base-256 digits the kernels carry per activation
# One registry and one set of workspaces per process, and ctypes releases the GIL during a call: callers are serialised.
_CUDA_LOCK = threading.RLock()


class CudaUnavailableError(RuntimeError):
    """The CUDA library is not built or no GPU is usable; there is no fallback path."""


class CudaRegistrationError(RuntimeError):
    """A resident weight could not be committed to device memory."""


class CudaContextError(RuntimeError):
    """A resident call failed validation, allocation, or an exact-envelope guard."""


def _signatures():
    """name -> (argument types, result type) of every symbol include/iie_qk.h declares."""
    c_int, i64, u64, vp = ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_void_p
    P64, P32 = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int)
    return {
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
        "iie_attn_decode_batch_dev": ([vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, vp, c_int, c_int, c_int, c_int, i64, c_int, i64, vp, vp], c_int),
        "iie_attn_block_dev": ([i64, i64, vp, vp, vp, i64, vp, i64, vp, vp, c_int, c_int, c_int, c_int, i64, c_int, c_int, i64, vp], c_int),
        "iie_block_dev": ([i64, i64, i64, i64, vp, vp, vp, i64, vp, i64, vp, vp, c_int, c_int, c_int, c_int, i64, c_int, c_int, u64, i64,
                           vp, vp, vp], c_int),
        "iie_embed_dev": ([i64, vp, i64, c_int, vp, vp], c_int), "iie_set_attn_fused": ([c_int], None), "iie_set_attn_tile_tc": ([c_int], None), "iie_argmax_dev": ([vp, i64, vp, vp], c_int),
        "iie_embed_rows_dev": ([i64, vp, c_int, c_int, vp, vp], c_int), "iie_argmax_rows_dev": ([vp, i64, i64, vp, vp], c_int),
        "iie_route_dev": ([i64, c_int, vp, i64, c_int, c_int, vp, vp, vp], c_int),
        "iie_moe_experts_dev": ([i64, vp, i64, vp, vp, c_int, c_int, c_int, c_int, c_int, vp, vp], c_int),
        "iie_moe_block_host": ([i64, i64, vp, i64, c_int, c_int, u64, vp, vp, vp], c_int),
        "iie_moe_block_dev": ([i64, i64, vp, i64, c_int, c_int, u64, vp, vp, vp, vp], c_int),
        "qk_attention_bank_moe_configure": ([i64, c_int, c_int, c_int, i64, i64], c_int),
        "qk_attention_bank_moe_bind": ([i64, c_int, c_int, i64, i64, i64], c_int),
        "qk_attention_bank_moe_begin": ([i64, c_int, i64, i64, i64, i64, i64, i64, vp, c_int, c_int, u64, c_int, c_int, i64, c_int,
                                         P32, P32], c_int),
        "qk_attention_bank_moe_continue": ([i64, c_int, c_int, c_int, i64, vp], c_int),
        "qk_attention_bank_moe_export": ([i64, i64, vp], c_int),
    }


# Every symbol the header declares; the CPU test-suite checks that the built library exports all of them.
EXPORTED_SYMBOLS = tuple(_signatures())


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libnmc_qk_cuda.so"


@lru_cache(maxsize=1)
def load_library():
    """``ctypes.CDLL`` of the in-tree library with argument types set; raises if it is not built.
    Loading needs no GPU (the CPU test-suite checks the exported symbols this way)."""
    path = lib_path()
    if not path.exists():
        raise CudaUnavailableError(f"{path} is not built (python -m integer_inference_engine_b200.build)")
    lib = ctypes.CDLL(str(path))
    table = _signatures()
    absent = [name for name in table if not hasattr(lib, name)]
    if absent:
        raise CudaUnavailableError(f"{path} lacks symbols {absent}")
    for name, (args, res) in table.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    return lib


def available() -> bool:
    """True when the library is built and a GPU is usable."""
    try:
        with _CUDA_LOCK:
            return load_library().qk_cuda_available() == 0
    except CudaUnavailableError:
        return False


def _lib():
    lib = load_library()
    with _CUDA_LOCK:
        usable = lib.qk_cuda_available() == 0
    if not usable:
        raise CudaUnavailableError("no usable CUDA device; this package has no CPU path")
    return lib


def _native(name: str, *args):
    """One native call under the lock."""
    fn = getattr(_lib(), name)
    with _CUDA_LOCK:
        return fn(*args)


# every optional capability of the reference bridge is always present in this library
resident_available = grouped_available = dp4a_available = resident_preprocess_available = available
moe_ffn_available = moe_ffn_dp4a_available = moe_ffn_batched_available = moe_ffn_batched_dp4a_available = available
resident_attention_available = resident_layer_available = available


# ------------------------------------------------------------------------------------------ argument helpers ---
def _rows(x) -> np.ndarray:
    """Activation as a C-contiguous int64 matrix; a vector is one row."""
    a = np.asarray(x, dtype=np.int64)
    if a.ndim < 2:
        a = a.reshape(1, -1)
    return np.ascontiguousarray(a)


def _blob(raw) -> np.ndarray:
    """Raw weight bytes as a uint8 array that stays alive for the duration of the call."""
    if isinstance(raw, np.ndarray):
        return np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    return np.frombuffer(raw, dtype=np.uint8)


def _require_weight_bytes(weight_raw, out_f: int, n_blocks: int, qtype: int) -> int:
    """Bytes the kernels will read for an [out_f, n_blocks*256] tensor of this type; a shorter buffer is refused here,
    before any pointer reaches native code."""
    if int(qtype) not in _BLOCK_BYTES:
        raise ValueError(f"qtype {qtype} is neither Q4_K ({Q4_K}) nor Q6_K ({Q6_K})")
    rows, blocks = int(out_f), int(n_blocks)
    if min(rows, blocks) <= 0:
        raise ValueError(f"a weight needs positive out_f and n_blocks, not {rows} and {blocks}")
    span = rows * blocks * _BLOCK_BYTES[int(qtype)]
    have = len(weight_raw)
    if have < span:
        raise ValueError(f"weight buffer holds {have} bytes, the tensor needs {span}")
    return span


def _handle_array(handles, n: int):
    return (ctypes.c_int64 * n)(*(int(h) for h in handles))


# --------------------------------------------------------------------------------------- products, residency ---
def qk_linear(weight_raw, x_int, out_f: int, n_blocks: int, fw: int, qtype: int):
    """y[t,o] = (sum_i W[o,i] x[t,i]) >> fw straight from raw Q4_K / Q6_K bytes: x [T, n_blocks*256] int64 -> [T, out_f].
    ``None`` when native code reports a failure."""
    x = _rows(x_int)
    if x.shape[1] != int(n_blocks) * 256:
        raise ValueError(f"activation width {x.shape[1]} does not match {n_blocks} blocks of 256")
    _require_weight_bytes(weight_raw, out_f, n_blocks, qtype)
    w = _blob(weight_raw)
    y = np.empty((x.shape[0], int(out_f)), np.int64)
    rc = _native("qk_linear_cuda", w.ctypes.data, x.ctypes.data, x.shape[0], int(out_f), int(n_blocks), int(fw), int(qtype),
                 y.ctypes.data)
    return y if rc == 0 else None


def register_weight(weight_raw, out_f: int, n_blocks: int, qtype: int) -> int:
    """Commit a Q4_K / Q6_K tensor to device memory once and return its handle."""
    _require_weight_bytes(weight_raw, out_f, n_blocks, qtype)
    w = _blob(weight_raw)
    handle = int(_native("qk_register_weight", w.ctypes.data, int(out_f), int(n_blocks), int(qtype)))
    if handle < 0:
        raise CudaRegistrationError(f"could not register a [{out_f}, {int(n_blocks) * 256}] tensor of qtype {qtype}")
    return handle


def register_i64(matrix) -> int:
    """Commit a dense int64 matrix (RMSNorm gain row, dense router); a vector counts as one row."""
    m = _rows(matrix)
    if m.ndim != 2 or 0 in m.shape:
        raise ValueError("a dense registration needs a non-empty vector or matrix")
    handle = int(_native("qk_register_i64", m.ctypes.data, m.shape[0], m.shape[1]))
    if handle < 0:
        raise CudaRegistrationError(f"could not register a dense int64 matrix of shape {m.shape}")
    return handle


def reserve_resident_capacity(count: int) -> bool:
    return _native("qk_resident_reserve", int(count)) == 0


def resident_count() -> int:
    return int(_native("qk_resident_count"))


def resident_capacity() -> int:
    return int(_native("qk_resident_capacity"))


def free_all() -> None:
    _native("qk_free_all")


def apply_resident(handle: int, x_int, out_f: int, fw: int):
    """x through a registered weight; ``None`` for an unknown handle or a native failure."""
    x = _rows(x_int)
    y = np.empty((x.shape[0], int(out_f)), np.int64)
    rc = _native("qk_apply_resident", int(handle), x.ctypes.data, x.shape[0], int(fw), y.ctypes.data)
    return y if rc == 0 else None


def apply_resident_grouped(handles, x_int, out_features, fw: int, phase_ids=None):
    """One activation through up to sixteen registered weights with a single upload and download; a tuple of results in
    the order of ``handles``.  ``phase_ids`` label the products for the profile counters."""
    hs, widths = [int(h) for h in handles], [int(n) for n in out_features]
    n = len(hs)
    if not 1 <= n <= _MAX_GROUP or len(widths) != n or min(widths) <= 0:
        raise ValueError(f"a grouped apply takes 1..{_MAX_GROUP} handles with one positive output width each")
    labels = [PROFILE_OTHER] * n if phase_ids is None else [int(p) for p in phase_ids]
    if len(labels) != n or not set(labels) <= {PROFILE_OTHER, PROFILE_Q, PROFILE_K, PROFILE_V, PROFILE_O}:
        raise ValueError("phase_ids must give one known phase label per handle")
    x = _rows(x_int)
    t = x.shape[0]
    packed = np.empty(t * sum(widths), np.int64)
    rc = _native("qk_apply_resident_grouped", _handle_array(hs, n), (ctypes.c_int * n)(*labels), n, x.ctypes.data, t, int(fw),
                 packed.size, packed.ctypes.data)
    if rc != 0:
        return None
    edges = np.cumsum([t * w for w in widths])[:-1]
    return tuple(part.reshape(t, w) for part, w in zip(np.split(packed, edges), widths))


# ------------------------------------------------------------------------------------------------ limb policy ---
def _balanced_capacity(L: int) -> int:
    """Largest magnitude L balanced base-256 digits (each in [-128, 127]) can represent."""
    return 127 * sum(256 ** i for i in range(int(L)))


_CAPACITY = [_balanced_capacity(L) for L in range(_DIGITS + 1)]


def limbs_needed(maxabs: int) -> int:
    """Fewest digits (1..8) that cover +-maxabs; OverflowError when even eight do not."""
    m = int(maxabs)
    for L in range(1, _DIGITS + 1):
        if m <= _CAPACITY[L]:
            return L
    raise OverflowError(f"magnitude {m} is beyond {_DIGITS} balanced base-256 digits ({_CAPACITY[_DIGITS]})")


def _activation_absmax(x: np.ndarray) -> int:
    return 0 if x.size == 0 else max(-int(x.min()), int(x.max()))


def _dp4a_limb_count(x: np.ndarray, requested=None):
    """Digit count handed to the type-specific applies.  The kernels always carry eight digits and recombine in 128 bits,
    so any sufficient count is exact.  ``None``: the activation needs a ninth digit and no count was asked for (the caller
    then uses :func:`apply_resident`, which takes the 128-bit kernel); an explicit count that cannot hold the activation is
    the caller's error."""
    try:
        need = limbs_needed(_activation_absmax(x))
    except OverflowError:
        if requested is None:
            return None
        raise ValueError(f"the activation does not fit {_DIGITS} balanced base-256 digits") from None
    if requested is None:
        return need
    want = int(requested)
    if want < 1 or want > _DIGITS:
        raise ValueError(f"a digit count lies in 1..{_DIGITS}, not {want}")
    if want < need:
        raise ValueError(f"{want} digits cannot hold this activation, which needs {need}")
    return want


def apply_resident_dp4a(handle: int, x_int, out_f: int, fw: int, qtype: int, ln=None):
    """Type-checked apply (same bytes as :func:`apply_resident`): ``None`` when the handle is of the other type or the
    activation needs a ninth digit."""
    entry = {Q4_K: "qk_apply_resident_q4k_dp4a", Q6_K: "qk_apply_resident_q6k_dp4a"}.get(qtype)
    if entry is None:
        raise ValueError(f"qtype {qtype} is neither Q4_K ({Q4_K}) nor Q6_K ({Q6_K})")
    x = _rows(x_int)
    digits = _dp4a_limb_count(x, ln)
    if digits is None:
        return None
    y = np.empty((x.shape[0], int(out_f)), np.int64)
    rc = _native(entry, int(handle), x.ctypes.data, x.shape[0], int(fw), digits, y.ctypes.data)
    return y if rc == 0 else None


def apply_resident_q6k_dp4a(handle: int, x_int, out_f: int, fw: int, ln=None):
    return apply_resident_dp4a(handle, x_int, out_f, fw, Q6_K, ln)


# ----------------------------------------------------------------------------------------- router, MoE block ---
def _rmsnorm_i128_safe(x: np.ndarray) -> bool:
    """Whether every row's sum of squares stays below 2**127, the width the native accumulator has."""
    if x.ndim != 2 or x.shape[1] == 0:
        return False
    limit = 1 << 127
    peak = np.abs(x.astype(object)).max(axis=1)                 # Python integers: abs(INT64_MIN) must not wrap
    for row, m in zip(x, peak):
        if int(m) ** 2 * x.shape[1] < limit:                    # the cheap bound settles almost every row
            continue
        if sum(int(v) * int(v) for v in row) >= limit:
            return False
    return True


def rmsnorm_router(gain_handle: int, router_handle: int, x_int, n_used: int, fa: int, fw: int, eps: int = 1):
    """Exact RMSNorm, dense int64 router product, top-k (lowest index wins ties), sigmoid gates.
    (h [T,D], ids [T,K] int32, gates [T,K]) or ``None`` when a row leaves the exact envelope; a bad shape or a runtime
    failure raises."""
    x = _rows(x_int)
    if 0 in x.shape:
        raise ValueError("the router needs a non-empty activation")
    k, fa, fw, eps = int(n_used), int(fa), int(fw), int(eps)
    if k <= 0:
        raise ValueError("n_used must be positive")
    if not (1 <= fa <= 29 and 0 <= fw <= 62 and 0 <= eps < 1 << 64):
        raise ValueError("fa, fw or eps lies outside what the native entry accepts")
    if not _rmsnorm_i128_safe(x):
        return None
    t = x.shape[0]
    h, ids, gates = np.empty_like(x), np.empty((t, k), np.int32), np.empty((t, k), np.int64)
    rc = int(_native("qk_rmsnorm_router", int(gain_handle), int(router_handle), x.ctypes.data, t, fa, fw, eps, k, h.size, ids.size,
                     h.ctypes.data, ids.ctypes.data, gates.ctypes.data))
    if rc == 3:
        return None
    if rc:
        raise CudaContextError(f"RMSNorm + router returned native status {rc}")
    return h, ids, gates


def _expert_triples(gate_h, up_h, down_h, count: int, what: str):
    if count <= 0 or not (len(gate_h) == len(up_h) == len(down_h) == count):
        raise ValueError(f"{what} needs {max(count, 1)} gate, up and down handles each")
    return tuple(_handle_array(hs, count) for hs in (gate_h, up_h, down_h))


def moe_ffn(gate_h, up_h, down_h, h, gates, d_model: int, e_ffn: int, fa: int, fw: int, dp4a: bool = False):
    """One token through its routed experts: out[d_model] = sum_e ((down_e(silu(gate_e h) * up_e h) * g_e) >> fa).
    ``dp4a`` selects the second entry name of the ABI; both give the same bytes.  ``None`` on a native failure."""
    n_e = len(gate_h)
    triples = _expert_triples(gate_h, up_h, down_h, n_e, "the expert stage")
    row, g = _rows(h).reshape(-1), _rows(gates).reshape(-1)
    if row.size != int(d_model) or g.size != n_e:
        raise ValueError(f"expected {d_model} hidden values and {n_e} gates, got {row.size} and {g.size}")
    out = np.empty(int(d_model), np.int64)
    rc = _native("qk_moe_ffn_dp4a" if dp4a else "qk_moe_ffn", *triples, n_e, row.ctypes.data, g.ctypes.data, int(d_model), int(e_ffn),
                 int(fa), int(fw), out.ctypes.data)
    return out if rc == 0 else None


def moe_ffn_batched(gate_h, up_h, down_h, m: int, k: int, h, gates, d_model: int, e_ffn: int, fa: int, fw: int, *,
                    dp4a: bool = False):
    """All m*k (token, routed expert) pairs in one call, handles flattened token-major (pair = t*k + j):
    h [m, d_model], gates [m*k] -> [m, d_model].  Prefill-sized calls run on the grouped tensor-core tiles."""
    m, k = int(m), int(k)
    if m <= 0 or k <= 0:
        raise ValueError(f"m and k must be positive, got {m} and {k}")
    pairs = m * k
    triples = _expert_triples(gate_h, up_h, down_h, pairs, "the batched expert stage")
    rows, g = _rows(h).reshape(-1), _rows(gates).reshape(-1)
    if rows.size != m * int(d_model) or g.size != pairs:
        raise ValueError(f"expected {m * int(d_model)} hidden values and {pairs} gates, got {rows.size} and {g.size}")
    out = np.empty((m, int(d_model)), np.int64)
    args = (*triples, m, k, rows.ctypes.data, g.ctypes.data, int(d_model), int(e_ffn), int(fa), int(fw), out.ctypes.data)
    rc = 2
    if dp4a and _dp4a_limb_count(rows) is not None and limbs_needed(_activation_absmax(rows)) <= 4:
        rc = _native("qk_moe_ffn_batched_dp4a", *args)              # status 2 = envelope miss: the exact entry follows
    if rc == 2:
        rc = _native("qk_moe_ffn_batched", *args)
    return out if rc == 0 else None


def moe_workspace_allocations() -> int:
    return int(_native("qk_moe_workspace_allocations"))


def moe_workspace_bytes() -> int:
    return int(_native("qk_moe_workspace_bytes"))


def release_moe_workspace() -> bool:
    _native("qk_moe_workspace_release")
    return True


def moe_block(layer_handle: int, x_int, n_used: int, fa: int, fw: int, gain_handle: int = -1, eps: int = 1):
    """Whole MoE block on host arrays in one native call: ``moe(x)`` or, with a gain handle, ``x + moe(rmsnorm(x, gain))``.
    (out [T,d], ids [T,k] int32, gates [T,k]) or ``None`` when an input leaves the exact envelope.  An additive entry
    without a counterpart in the reference bridge: one upload and one download instead of the per-layer sequence
    rmsnorm_router + moe_ffn."""
    x = _rows(x_int)
    t, k = x.shape[0], int(n_used)
    out, ids, gates = np.empty_like(x), np.empty((t, k), np.int32), np.empty((t, k), np.int64)
    rc = _native("iie_moe_block_host", int(layer_handle), int(gain_handle), x.ctypes.data, t, int(fa), int(fw), int(eps),
                 out.ctypes.data, ids.ctypes.data, gates.ctypes.data)
    if rc == 3:
        return None
    if rc:
        raise CudaContextError(f"the MoE block returned native status {rc}")
    return out, ids, gates


# ------------------------------------------------------------------------------------------- profile counters ---
def profile_reset(*, enabled: bool = True) -> bool:
    """Zero the native counters; collection is on afterwards unless ``enabled`` is false."""
    lib = _lib()
    with _CUDA_LOCK:                                 # one critical section: no call may count between the three steps
        lib.qk_profile_set_enabled(0)
        lib.qk_profile_reset()
        lib.qk_profile_set_enabled(1 if enabled else 0)
    return True


def profile_set_enabled(enabled: bool) -> bool:
    _native("qk_profile_set_enabled", 1 if enabled else 0)
    return True


def profile_snapshot() -> dict:
    n = len(_PROFILE_METRICS)
    raw = (ctypes.c_uint64 * n)()
    if _native("qk_profile_snapshot", raw, n) != n:
        raise CudaContextError("the native profile snapshot has an unexpected number of counters")
    return dict(zip(_PROFILE_METRICS, (int(v) for v in raw)))


# --------------------------------------------------------------------------------------------- attention bank ---
class ResidentAttentionCache:
    """K/V rows of one request kept on the device, and the single-token attention sublayer over them
    (``qk_attention_bank_*``).  After a prefill each layer's K/V is imported once; every :meth:`apply` takes one
    normalised hidden row, appends that token's K/V row on the device and returns the projected attention row.
    A call that fails leaves its layer unusable: the caller drops the context rather than retrying."""

    def __init__(self, n_layers: int, max_length: int, d_model: int, n_heads: int, n_kv: int, head_dim: int, fa: int, cos, sin):
        dims = dict(n_layers=int(n_layers), max_length=int(max_length), d_model=int(d_model), n_heads=int(n_heads),
                    n_kv=int(n_kv), head_dim=int(head_dim), fa=int(fa))
        q_width = dims["n_heads"] * dims["head_dim"]
        positive = all(dims[name] > 0 for name in ("n_layers", "max_length", "d_model", "n_heads", "n_kv", "head_dim"))
        if not positive or dims["n_heads"] % dims["n_kv"] or dims["head_dim"] % 2 or dims["d_model"] % 256 or q_width % 256 \
                or not 1 <= dims["fa"] <= 29:
            raise ValueError(f"the attention bank cannot take these dimensions: {dims}")
        tables = [np.ascontiguousarray(np.asarray(t, dtype=np.int64)) for t in (cos, sin)]
        want = (dims["max_length"], dims["head_dim"] // 2)
        if any(t.shape != want for t in tables):
            raise ValueError(f"cos and sin must each be {want}, got {tables[0].shape} and {tables[1].shape}")
        handle = int(_native("qk_attention_bank_create", dims["n_layers"], dims["max_length"], dims["d_model"], dims["n_heads"],
                             dims["n_kv"], dims["head_dim"], dims["fa"], tables[0].ctypes.data, tables[1].ctypes.data))
        if handle < 0:
            raise CudaContextError("the attention bank could not be created (dimensions or device memory)")
        self.handle, self.q_width = handle, q_width
        for name, value in dims.items():
            setattr(self, name, value)
        self._filled = [0] * dims["n_layers"]
        self._open = True
        self._moe_shape = {}              # layer -> (experts, used, e_ffn) as configured
        self._begun = None                # layer whose begin_moe_layer awaits its continue_moe_layer
        self._epoch = 0                   # advances whenever the retained row changes; markers of older epochs are stale

    def _check(self, layer: int) -> int:
        if not self._open:
            raise CudaContextError("this attention bank has been closed")
        layer = int(layer)
        if not 0 <= layer < self.n_layers:
            raise ValueError(f"layer {layer} is outside 0..{self.n_layers - 1}")
        return layer

    def length(self, layer=0):
        return self._filled[layer]

    def import_layer(self, layer: int, k, v) -> None:
        layer = self._check(layer)
        rows = [np.ascontiguousarray(np.asarray(t, dtype=np.int64)) for t in (k, v)]
        if rows[0].ndim != 3 or rows[0].shape != rows[1].shape or rows[0].shape[0] != self.n_kv or rows[0].shape[2] != self.head_dim:
            raise ValueError(f"K and V must both be [{self.n_kv}, length, {self.head_dim}]")
        filled = rows[0].shape[1]
        if filled > self.max_length:
            raise ValueError(f"{filled} rows do not fit a bank of {self.max_length}")
        if _native("qk_attention_bank_import", self.handle, layer, rows[0].ctypes.data, rows[1].ctypes.data, filled) != 0:
            raise CudaContextError(f"importing K/V into layer {layer} failed")
        self._filled[layer] = filled

    def apply(self, layer: int, q_handle: int, k_handle: int, v_handle: int, o_handle: int, hidden, fw: int,
              window: "int | None", rope: bool):
        layer = self._check(layer)
        if self._filled[layer] >= self.max_length:
            raise ValueError(f"layer {layer} already holds its {self.max_length} rows")
        x = np.ascontiguousarray(np.asarray(hidden, dtype=np.int64))
        if x.shape != (1, self.d_model):
            raise ValueError(f"the hidden row must be (1, {self.d_model}), not {x.shape}")
        out = np.empty_like(x)
        scale = int(round(2 ** self.fa / self.head_dim ** 0.5))
        rc = int(_native("qk_attention_bank_apply", self.handle, layer, int(q_handle), int(k_handle), int(v_handle), int(o_handle),
                         x.ctypes.data, int(fw), -1 if window is None else int(window), 1 if rope else 0, scale, out.size,
                         out.ctypes.data))
        if rc:
            why = "a value left the exact envelope" if rc == 3 else f"native status {rc}"
            raise CudaContextError(f"attention on layer {layer} failed: {why}")
        self._filled[layer] += 1
        return out

    # -- retained-layer executor: a token walks consecutive MoE layers with its residual row kept on the device --------
    def configure_moe_layer(self, layer: int, n_experts: int, n_used: int, d_model: int, expert_ffn: int) -> None:
        """Declare the expert table of one layer (no expert weight is touched; see :meth:`bind_moe_expert`)."""
        layer = self._check(layer)
        shape = (int(n_experts), int(n_used), int(expert_ffn))
        if int(d_model) != self.d_model or shape[0] <= 0 or not 0 < shape[1] <= shape[0] or shape[2] <= 0 or shape[2] % 256:
            raise ValueError(f"layer {layer}: not a usable MoE shape {shape} at width {d_model}")
        if self._moe_shape.get(layer, shape) != shape:
            raise ValueError(f"layer {layer} is already configured as {self._moe_shape[layer]}")
        if _native("qk_attention_bank_moe_configure", self.handle, layer, shape[0], shape[1], self.d_model, shape[2]) != 0:
            raise CudaContextError(f"the MoE table of layer {layer} could not be configured")
        self._moe_shape[layer] = shape

    def bind_moe_expert(self, layer: int, expert: int, gate_handle: int, up_handle: int, down_handle: int) -> None:
        """Let this request use the registered (gate, up, down) matrices as expert ``expert`` of ``layer``."""
        layer, expert = self._check(layer), int(expert)
        if layer not in self._moe_shape or not 0 <= expert < self._moe_shape[layer][0]:
            raise ValueError(f"expert {expert} of layer {layer} is outside the configured table")
        if _native("qk_attention_bank_moe_bind", self.handle, layer, expert, int(gate_handle), int(up_handle), int(down_handle)) != 0:
            raise CudaContextError(f"binding expert {expert} of layer {layer} failed")

    def begin_moe_layer(self, layer: int, gain_handle: int, router_handle: int, q_handle: int, k_handle: int, v_handle: int,
                        o_handle: int, hidden, fw: int, eps: int, window: "int | None", rope: bool) -> "tuple[int, ...]":
        """Norm, routing and the attention sublayer of one token on ``layer``; everything stays on the device.  ``hidden`` is a
        host row [1, d_model] or the marker a previous :meth:`continue_moe_layer` returned.  Returns the selected experts
        that are not bound yet: bind them, then call :meth:`continue_moe_layer`."""
        layer = self._check(layer)
        if layer not in self._moe_shape or self._begun is not None or self._filled[layer] >= self.max_length:
            raise ValueError(f"layer {layer} cannot begin: not configured, another layer is pending, or the bank is full")
        if isinstance(hidden, ResidentLayerHidden):
            if hidden.bank is not self or hidden.epoch != self._epoch:
                raise ValueError("this retained-row marker is stale or belongs to another bank")
            keep, pointer, retained = None, None, 1
        else:
            keep = np.ascontiguousarray(np.asarray(hidden, dtype=np.int64))
            if keep.shape != (1, self.d_model):
                raise ValueError(f"the hidden row must be (1, {self.d_model}), not {keep.shape}")
            pointer, retained = keep.ctypes.data, 0
        used = self._moe_shape[layer][1]
        count, cold = ctypes.c_int(0), (ctypes.c_int * used)()
        scale = int(round(2 ** self.fa / self.head_dim ** 0.5))
        rc = int(_native("qk_attention_bank_moe_begin", self.handle, layer, int(gain_handle), int(router_handle), int(q_handle),
                         int(k_handle), int(v_handle), int(o_handle), pointer, retained, int(fw), int(eps),
                         -1 if window is None else int(window), 1 if rope else 0, scale, used, ctypes.byref(count), cold))
        if rc:
            why = "a value left the exact envelope" if rc == 3 else f"native status {rc}"
            raise CudaContextError(f"begin on layer {layer} failed: {why}")
        if not 0 <= count.value <= used:
            raise CudaContextError(f"layer {layer} reported {count.value} cold experts of {used} selected")
        self._filled[layer] += 1
        self._begun = layer
        return tuple(int(cold[i]) for i in range(count.value))

    def continue_moe_layer(self, layer: int, fw: int, *, publish: bool = False):
        """Expert stage and residual of the layer begun last.  Returns the new residual row (``publish``) or a marker that
        only the next layer's :meth:`begin_moe_layer` of this bank accepts."""
        layer = self._check(layer)
        if self._begun != layer:
            raise ValueError(f"layer {layer} has no begin_moe_layer pending")
        out = np.empty((1, self.d_model), dtype=np.int64) if publish else None
        rc = int(_native("qk_attention_bank_moe_continue", self.handle, layer, int(fw), 1 if publish else 0,
                         0 if out is None else out.size, None if out is None else out.ctypes.data))
        if rc:
            why = {3: "a value left the exact envelope", 4: "selected cold experts remain unbound"}.get(rc, f"native status {rc}")
            raise CudaContextError(f"continue on layer {layer} failed: {why}")
        self._begun = None
        self._epoch += 1
        return out if publish else ResidentLayerHidden(self, self._epoch)

    def export_moe_hidden(self) -> np.ndarray:
        """Copy of the retained residual row (debugging, or leaving the retained chain early)."""
        if not self._open or self._begun is not None:
            raise CudaContextError("no retained row can be exported while the bank is closed or a layer is pending")
        out = np.empty((1, self.d_model), dtype=np.int64)
        if _native("qk_attention_bank_moe_export", self.handle, out.size, out.ctypes.data) != 0:
            raise CudaContextError("the bank holds no retained row")
        return out

    def reset(self) -> None:
        if not self._open:
            raise CudaContextError("this attention bank has been closed")
        if _native("qk_attention_bank_reset", self.handle) != 0:
            raise CudaContextError("the attention bank could not be reset")
        self._filled = [0] * self.n_layers
        self._begun = None
        self._epoch += 1

    def workspace_bytes(self) -> int:
        if not self._open:
            raise CudaContextError("this attention bank has been closed")
        value = int(_native("qk_attention_bank_workspace_bytes", self.handle))
        if value == 2 ** 64 - 1:
            raise CudaContextError("the bank could not account for its device memory")
        return value

    def close(self) -> None:
        if self._open:
            _native("qk_attention_bank_destroy", self.handle)
            self._open = False
            self._begun = None
            self._epoch += 1

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class ResidentLayerHidden:
    """Stands for the residual row a bank keeps on the device after ``continue_moe_layer(publish=False)``."""
    __slots__ = ("bank", "epoch")

    def __init__(self, bank: ResidentAttentionCache, epoch: int):
        self.bank, self.epoch = bank, epoch


class ResidentMoeLayerSpec:
    """Handles and attention settings of one MoE layer of a retained chain."""
    __slots__ = ("layer", "gain_handle", "router_handle", "q_handle", "k_handle", "v_handle", "o_handle", "window", "rope")

    def __init__(self, layer, gain_handle, router_handle, q_handle, k_handle, v_handle, o_handle, window, rope):
        self.layer, self.gain_handle, self.router_handle = int(layer), int(gain_handle), int(router_handle)
        self.q_handle, self.k_handle, self.v_handle, self.o_handle = int(q_handle), int(k_handle), int(v_handle), int(o_handle)
        self.window, self.rope = (None if window is None else int(window)), bool(rope)


class ResidentMoeTokenExecutor:
    """One decode token through ``layer_count`` consecutive MoE layers of a bank, uploading only the experts a token selects
    (north-mini-code/src/nmc/qk_cuda.py:741-867).  ``lookup_expert(layer, expert)`` returns the (gate, up, down) handles of an
    expert that is already registered, or ``None``; ``load_expert(layer, expert)`` registers one and returns its handles, and
    is called only for the experts a layer reports as cold.  After any failure the executor refuses further work: the K/V
    rows of the layers already visited have advanced, so the request has to be reset or dropped."""

    def __init__(self, cache: ResidentAttentionCache, *, first_layer: int, layer_count: int, n_experts: int, n_used: int,
                 d_model: int, expert_ffn: int, fw: int, eps: int, lookup_expert, load_expert):
        if not isinstance(cache, ResidentAttentionCache) or not cache._open:
            raise ValueError("the executor needs an open attention bank")
        if not callable(lookup_expert) or not callable(load_expert):
            raise TypeError("lookup_expert and load_expert must be callables")
        self.first_layer, self.layer_count = int(first_layer), int(layer_count)
        self.shape = (int(n_experts), int(n_used), int(d_model), int(expert_ffn))
        self.fw, self.eps = int(fw), int(eps)
        last = self.first_layer + self.layer_count
        if self.first_layer < 0 or self.layer_count <= 0 or last > cache.n_layers or self.shape[0] <= 0 or \
                not 0 < self.shape[1] <= self.shape[0] or self.shape[2] != cache.d_model or self.shape[3] <= 0 or \
                self.shape[3] % 256 or not 0 <= self.fw <= 62 or not 0 <= self.eps < 2 ** 64:
            raise ValueError("the executor cannot take these dimensions")
        self.cache, self.lookup_expert, self.load_expert = cache, lookup_expert, load_expert
        self._tables_done = set()           # layers whose table is configured and whose known experts are bound
        self.poisoned = False

    @staticmethod
    def _triplet(value, where: str):
        try:
            handles = tuple(int(h) for h in value)
        except (TypeError, ValueError):
            handles = ()
        if len(handles) != 3 or min(handles, default=-1) < 0:
            raise CudaContextError(f"{where} did not give a (gate, up, down) handle triplet")
        return handles

    def _table(self, layer: int) -> None:
        if layer in self._tables_done:
            return
        experts, used, d_model, e_ffn = self.shape
        self.cache.configure_moe_layer(layer, experts, used, d_model, e_ffn)
        for expert in range(experts):
            known = self.lookup_expert(layer, expert)
            if known is not None:
                self.cache.bind_moe_expert(layer, expert, *self._triplet(known, f"lookup of expert {expert}, layer {layer}"))
        self._tables_done.add(layer)

    def _specs(self, layers):
        specs = tuple(layers)
        want = list(range(self.first_layer, self.first_layer + self.layer_count))
        if [getattr(spec, "layer", None) for spec in specs] != want or not all(isinstance(s, ResidentMoeLayerSpec) for s in specs):
            raise ValueError(f"the executor runs layers {want[0]}..{want[-1]} in order")
        return specs

    def prepare(self, layers):
        """Configure the tables and bind what is already resident, before any K/V row moves."""
        if self.poisoned:
            raise CudaContextError("this executor failed earlier: reset or drop the request")
        specs = self._specs(layers)
        try:
            for spec in specs:
                self._table(spec.layer)
        except Exception:
            self.poisoned = True
            raise
        return specs

    def run(self, hidden, layers) -> np.ndarray:
        specs = self.prepare(layers)
        row = np.ascontiguousarray(np.asarray(hidden, dtype=np.int64))
        if row.shape != (1, self.shape[2]):
            raise ValueError(f"the hidden row must be (1, {self.shape[2]}), not {row.shape}")
        try:
            state = row
            for spec in specs:
                cold = self.cache.begin_moe_layer(spec.layer, spec.gain_handle, spec.router_handle, spec.q_handle, spec.k_handle,
                                                  spec.v_handle, spec.o_handle, state, self.fw, self.eps, spec.window, spec.rope)
                if len(set(cold)) != len(cold) or any(not 0 <= e < self.shape[0] for e in cold):
                    raise CudaContextError(f"layer {spec.layer} reported cold experts {cold}")
                for expert in cold:
                    loaded = self._triplet(self.load_expert(spec.layer, expert), f"load of expert {expert}, layer {spec.layer}")
                    self.cache.bind_moe_expert(spec.layer, expert, *loaded)
                state = self.cache.continue_moe_layer(spec.layer, self.fw, publish=spec is specs[-1])
            if not isinstance(state, np.ndarray):
                raise CudaContextError("the last layer did not publish its row")
            return state
        except Exception:
            self.poisoned = True
            raise
