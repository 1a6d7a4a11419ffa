"""ctypes access to the compiled CPU checkers.  TEST INFRASTRUCTURE ONLY.

``orc`` wraps ``oracle/_build/liborc.so`` (this repository's C restatement); ``ref_qk_linear`` calls
the reference project's own ``qk_linear`` from ``oracle/_ref/libnmc_qk.so`` when that was built.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

import numpy as np

from . import build

HERE = Path(__file__).resolve().parent
_P = ctypes.c_void_p
_I64 = ctypes.c_int64


@lru_cache(maxsize=1)
def orc():
    lib = ctypes.CDLL(str(build.build_oracle()))
    lib.orc_half_to_fixed.argtypes = [ctypes.c_uint16, ctypes.c_int]
    lib.orc_half_to_fixed.restype = _I64
    lib.orc_qk_linear.argtypes = [_P, _P, _I64, _I64, _I64, ctypes.c_int, ctypes.c_int, _P]
    lib.orc_qk_linear.restype = None
    lib.orc_sigmoid_vec.argtypes = [_P, _I64, ctypes.c_int, _P]
    lib.orc_silu_vec.argtypes = [_P, _I64, ctypes.c_int, _P]
    lib.orc_topk_lowidx.argtypes = [_P, ctypes.c_int, ctypes.c_int, _P]
    lib.orc_moe_block.argtypes = [_P, ctypes.c_int, _P, _P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                  ctypes.c_int, _P, _I64, _I64, _I64, ctypes.c_int, ctypes.c_int, _P, _P, _P, _P]
    lib.orc_moe_block.restype = None
    lib.orc_q1_linear.argtypes = [_P, _P, _P, _I64, _I64, _I64, ctypes.c_int, _P]
    lib.orc_q1_linear.restype = None
    return lib


def _raw(buf) -> np.ndarray:
    return np.frombuffer(buf, np.uint8) if not isinstance(buf, np.ndarray) else np.ascontiguousarray(buf).view(np.uint8).reshape(-1)


def qk_linear(raw, x, out_f: int, n_blocks: int, fw: int, qtype: int) -> np.ndarray:
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x, np.int64)))
    w = _raw(raw)
    out = np.empty((x.shape[0], out_f), np.int64)
    orc().orc_qk_linear(w.ctypes.data, x.ctypes.data, x.shape[0], out_f, n_blocks, fw, qtype, out.ctypes.data)
    return out


def sigmoid(x, fa: int = 16) -> np.ndarray:
    x = np.ascontiguousarray(np.asarray(x, np.int64))
    out = np.empty_like(x)
    orc().orc_sigmoid_vec(x.ctypes.data, x.size, fa, out.ctypes.data)
    return out


def silu(x, fa: int = 16) -> np.ndarray:
    x = np.ascontiguousarray(np.asarray(x, np.int64))
    out = np.empty_like(x)
    orc().orc_silu_vec(x.ctypes.data, x.size, fa, out.ctypes.data)
    return out


def topk_lowidx(logits, k: int) -> np.ndarray:
    v = np.ascontiguousarray(np.asarray(logits, np.int64))
    ids = np.empty(k, np.int32)
    orc().orc_topk_lowidx(v.ctypes.data, v.size, k, ids.ctypes.data)
    return ids


def moe_block(router_raw, router_qtype, gate_raws, up_raws, down_raws, gate_qtype, down_qtype, k, h,
              d_model: int, e_ffn: int, fa: int, fw: int):
    """Whole MoE FFN on the CPU.  Weight arguments are sequences of raw per-expert tensors.
    Returns (ids [T,k] int32, gates [T,k] int64, out [T,d_model] int64)."""
    h = np.ascontiguousarray(np.atleast_2d(np.asarray(h, np.int64)))
    T, n_e = h.shape[0], len(gate_raws)
    keep = [[_raw(b) for b in lst] for lst in (gate_raws, up_raws, down_raws)]
    tabs = [(ctypes.c_void_p * n_e)(*[a.ctypes.data for a in lst]) for lst in keep]
    r = _raw(router_raw)
    ids = np.empty((T, k), np.int32); gates = np.empty((T, k), np.int64); out = np.empty((T, d_model), np.int64)
    scratch = np.empty(T * n_e + 2 * e_ffn + d_model, np.int64)
    orc().orc_moe_block(r.ctypes.data, router_qtype, tabs[0], tabs[1], tabs[2], gate_qtype, down_qtype, n_e, k,
                        h.ctypes.data, T, d_model, e_ffn, fa, fw, ids.ctypes.data, gates.ctypes.data,
                        out.ctypes.data, scratch.ctypes.data)
    return ids, gates, out


def q1_linear(x, bits, scale, frac: int) -> np.ndarray:
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x, np.int64)))
    b = np.ascontiguousarray(np.asarray(bits, np.uint8)); s = np.ascontiguousarray(np.asarray(scale, np.int64))
    out_f, nb = s.shape
    out = np.empty((x.shape[0], out_f), np.int64)
    orc().orc_q1_linear(x.ctypes.data, b.ctypes.data, s.ctypes.data, x.shape[0], out_f, nb, frac, out.ctypes.data)
    return out


@lru_cache(maxsize=1)
def _ref():
    p = HERE / "_ref" / "libnmc_qk.so"
    if not p.exists():
        build.build_ref()
    if not p.exists():
        return None
    lib = ctypes.CDLL(str(p))
    lib.qk_linear.argtypes = [_P, _P, _I64, _I64, _I64, ctypes.c_int, ctypes.c_int, _P]
    lib.qk_linear.restype = None
    return lib


def ref_available() -> bool:
    return _ref() is not None


def ref_qk_linear(raw, x, out_f: int, n_blocks: int, fw: int, qtype: int) -> np.ndarray:
    """The reference project's compiled CPU kernel (north-mini-code/tools/nmc_qk_kernel.c:85)."""
    lib = _ref()
    x = np.ascontiguousarray(np.atleast_2d(np.asarray(x, np.int64)))
    w = _raw(raw)
    out = np.empty((x.shape[0], out_f), np.int64)
    lib.qk_linear(w.ctypes.data, x.ctypes.data, x.shape[0], out_f, n_blocks, fw, qtype, out.ctypes.data)
    return out
