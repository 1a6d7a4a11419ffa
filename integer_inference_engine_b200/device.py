"""Device-tensor front end: the MoE block on PyTorch CUDA tensors, no host round trip.

PyTorch only owns memory and streams here; all arithmetic runs in ``libnmc_qk_cuda.so`` through the
device-pointer entry points of the C-ABI (``iie_*`` in include/iie_qk.h).  The composition follows
``Engine._moe`` of the reference (north-mini-code/src/nmc/engine.py:375-443): router product, top-k
with lowest-index tie-break, sigmoid gates, per-expert gate/up products, integer SiLU, down
product, one floor per expert term and an exact sum.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import qk_cuda
from .qk_cuda import Q4_K, Q6_K, _BLOCK_BYTES, _CUDA_LOCK, CudaContextError, CudaRegistrationError


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def register_weight(raw, out_f: int, n_blocks: int, qtype: int) -> int:
    """Register raw Q4_K / Q6_K blocks held in a CUDA uint8 tensor, a NumPy array or bytes."""
    lib = qk_cuda._lib()
    need = out_f * n_blocks * _BLOCK_BYTES[qtype]
    if isinstance(raw, torch.Tensor):
        if not raw.is_cuda or raw.dtype != torch.uint8 or not raw.is_contiguous() or raw.numel() < need:
            raise ValueError("raw weight tensor must be a contiguous CUDA uint8 tensor of the full size")
        torch.cuda.current_stream().synchronize()        # the library copies on its own stream
        with _CUDA_LOCK:
            h = lib.iie_register_weight_dev(raw.data_ptr(), out_f, n_blocks, qtype)
        if h < 0:
            raise CudaRegistrationError(f"device registration failed for [{out_f}, {n_blocks * 256}] qtype {qtype}")
        return int(h)
    return qk_cuda.register_weight(raw, out_f, n_blocks, qtype)


def export_weight(handle: int, out_f: int, n_blocks: int, qtype: int) -> np.ndarray:
    """Raw GGUF-order bytes of a registered weight (for checking against a CPU oracle)."""
    lib = qk_cuda._lib()
    buf = np.empty(out_f * n_blocks * _BLOCK_BYTES[qtype], np.uint8)
    with _CUDA_LOCK:
        rc = lib.iie_weight_export(int(handle), buf.ctypes.data)
    if rc != 0:
        raise CudaContextError(f"weight export failed with status {rc}")
    return buf


def apply(handle: int, x: torch.Tensor, out_f: int, fw: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """out [T,out_f] = floor(x W^T / 2^fw) for a registered weight, on the current stream."""
    lib = qk_cuda._lib()
    x = x.contiguous()
    assert x.is_cuda and x.dtype == torch.int64 and x.dim() == 2
    if out is None:
        out = torch.empty((x.shape[0], out_f), dtype=torch.int64, device=x.device)
    assert out.is_contiguous() and out.numel() == x.shape[0] * out_f
    with _CUDA_LOCK:
        rc = lib.iie_apply_dev(int(handle), x.data_ptr(), x.shape[0], int(fw), out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"device apply failed with status {rc}")
    return out


def rmsnorm(x: torch.Tensor, gain_handle: int = -1, fa: int = 16, eps: int = 1, out: torch.Tensor | None = None):
    """Integer RMSNorm of x [rows,width] with an optional registered int64 gain row."""
    lib = qk_cuda._lib()
    x = x.contiguous()
    assert x.is_cuda and x.dtype == torch.int64 and x.dim() == 2
    if out is None:
        out = torch.empty_like(x)
    with _CUDA_LOCK:
        rc = lib.iie_rmsnorm_dev(int(gain_handle), x.data_ptr(), x.shape[0], x.shape[1], int(fa), int(eps),
                                 out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"device RMSNorm failed with status {rc}")
    return out


def attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     pos: int, n_heads: int, n_kv: int, head_dim: int, fa: int = 16, window: int = 0,
                     cos: torch.Tensor | None = None, sin: torch.Tensor | None = None, rope: int = 0,
                     inv_sqrt: int | None = None, out: torch.Tensor | None = None,
                     pos_dev: torch.Tensor | None = None) -> torch.Tensor:
    """One new token's GQA attention over the int32 caches ``[n_kv, rows, head_dim]``; writes cache row ``pos``
    (``q`` and ``k`` are given before rotation and are not modified).  With ``pos_dev`` (CUDA int32 [1]) the position is read on the device and ``pos``
    is an upper bound (for replayed graphs).  Returns ``[n_heads * head_dim]`` int64."""
    lib = qk_cuda._lib()
    assert q.is_cuda and q.dtype == torch.int64 and q.is_contiguous() and q.numel() == n_heads * head_dim
    assert k.dtype == torch.int64 and v.dtype == torch.int64 and k.numel() == n_kv * head_dim == v.numel()
    assert kcache.dtype == torch.int32 and vcache.dtype == torch.int32 and kcache.is_contiguous() and vcache.is_contiguous()
    assert kcache.shape == vcache.shape and kcache.shape[0] == n_kv and kcache.shape[2] == head_dim
    if inv_sqrt is None:
        inv_sqrt = int(round((1.0 / head_dim ** 0.5) * (1 << fa)))
    if out is None:
        out = torch.empty(n_heads * head_dim, dtype=torch.int64, device=q.device)
    with _CUDA_LOCK:
        rc = lib.iie_attn_decode_dev(q.data_ptr(), k.contiguous().data_ptr(), v.contiguous().data_ptr(), kcache.data_ptr(),
                                     vcache.data_ptr(), int(pos), pos_dev.data_ptr() if pos_dev is not None else None,
                                     int(window or 0), cos.data_ptr() if rope else None,
                                     sin.data_ptr() if rope else None, int(rope), n_heads, n_kv, head_dim,
                                     int(kcache.shape[1]), int(fa), int(inv_sqrt), out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"attention failed with status {rc}")
    return out


def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, start: int,
                      n_heads: int, n_kv: int, head_dim: int, fa: int = 16, window: int = 0, cos: torch.Tensor | None = None,
                      sin: torch.Tensor | None = None, rope: int = 0, inv_sqrt: int | None = None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of ``m`` new tokens at positions ``start .. start + m - 1``: ``q`` [m, n_heads*head_dim], ``k`` / ``v``
    [m, n_kv*head_dim] before rotation; writes their cache rows, returns ``[m, n_heads*head_dim]`` int64."""
    lib = qk_cuda._lib()
    m = q.shape[0]
    assert q.is_cuda and q.dtype == torch.int64 and q.is_contiguous() and q.shape[1] == n_heads * head_dim
    assert k.dtype == torch.int64 and v.dtype == torch.int64 and k.is_contiguous() and v.is_contiguous()
    assert k.shape == (m, n_kv * head_dim) == v.shape
    assert kcache.dtype == torch.int32 and vcache.dtype == torch.int32 and kcache.is_contiguous() and vcache.is_contiguous()
    assert kcache.shape == vcache.shape and kcache.shape[0] == n_kv and kcache.shape[2] == head_dim
    if inv_sqrt is None:
        inv_sqrt = int(round((1.0 / head_dim ** 0.5) * (1 << fa)))
    if out is None:
        out = torch.empty((m, n_heads * head_dim), dtype=torch.int64, device=q.device)
    with _CUDA_LOCK:
        rc = lib.iie_attn_prefill_dev(q.data_ptr(), k.data_ptr(), v.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), int(start), int(m),
                                      int(window or 0), cos.data_ptr() if rope else None, sin.data_ptr() if rope else None, int(rope),
                                      n_heads, n_kv, head_dim, int(kcache.shape[1]), int(fa), int(inv_sqrt), out.data_ptr(),
                                      _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"prefill attention failed with status {rc}")
    return out


def attention_decode_batch(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: int,
                           n_heads: int, n_kv: int, head_dim: int, fa: int = 16, window: int = 0, cos: torch.Tensor | None = None,
                           sin: torch.Tensor | None = None, rope: int = 0, inv_sqrt: int | None = None,
                           out: torch.Tensor | None = None) -> torch.Tensor:
    """The new tokens of ``B`` independent sequences, all at position ``pos``: ``q`` [B, n_heads*head_dim], ``k`` / ``v``
    [B, n_kv*head_dim] before rotation, caches [B, n_kv, rows, head_dim] int32 (row ``pos`` of each is written).
    Returns [B, n_heads*head_dim] int64."""
    lib = qk_cuda._lib()
    B = q.shape[0]
    assert q.is_cuda and q.dtype == torch.int64 and q.is_contiguous() and q.shape == (B, n_heads * head_dim)
    assert k.dtype == torch.int64 and v.dtype == torch.int64 and k.is_contiguous() and v.is_contiguous()
    assert k.shape == (B, n_kv * head_dim) == v.shape
    assert kcache.dtype == torch.int32 and vcache.dtype == torch.int32 and kcache.is_contiguous() and vcache.is_contiguous()
    assert kcache.shape == vcache.shape and kcache.shape[0] == B and kcache.shape[1] == n_kv and kcache.shape[3] == head_dim
    if inv_sqrt is None:
        inv_sqrt = int(round((1.0 / head_dim ** 0.5) * (1 << fa)))
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.int64, device=q.device)
    with _CUDA_LOCK:
        rc = lib.iie_attn_decode_batch_dev(q.data_ptr(), k.data_ptr(), v.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), int(pos), B,
                                           int(kcache.stride(0)), int(window or 0), cos.data_ptr() if rope else None,
                                           sin.data_ptr() if rope else None, int(rope), n_heads, n_kv, head_dim,
                                           int(kcache.shape[2]), int(fa), int(inv_sqrt), out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"batched decode attention failed with status {rc}")
    return out


def attention_block(wqkv: int, wo: int, x: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: int, n_heads: int,
                    n_kv: int, head_dim: int, fa: int = 16, fw: int = 24, window: int = 0, cos: torch.Tensor | None = None,
                    sin: torch.Tensor | None = None, rope: int = 0, inv_sqrt: int | None = None,
                    pos_dev: torch.Tensor | None = None) -> None:
    """``x += attention(...) Wo^T`` for the row the last single-token MoE block call normalised (see
    ``iie_attn_block_dev``): fused QKV product, cache append, exact attention, O product."""
    lib = qk_cuda._lib()
    assert x.is_cuda and x.dtype == torch.int64 and x.is_contiguous()
    assert kcache.dtype == torch.int32 and vcache.dtype == torch.int32 and kcache.is_contiguous() and vcache.is_contiguous()
    if inv_sqrt is None:
        inv_sqrt = int(round((1.0 / head_dim ** 0.5) * (1 << fa)))
    with _CUDA_LOCK:
        rc = lib.iie_attn_block_dev(int(wqkv), int(wo), x.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), int(pos),
                                    pos_dev.data_ptr() if pos_dev is not None else None, int(window or 0),
                                    cos.data_ptr() if rope else None, sin.data_ptr() if rope else None, int(rope), n_heads, n_kv,
                                    head_dim, int(kcache.shape[1]), int(fa), int(fw), int(inv_sqrt), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"attention block failed with status {rc}")


class NoFusedBlock(RuntimeError):
    """The shape has no five-launch block form; use ``MoELayer.block`` followed by :func:`attention_block`."""


def decoder_block(layer: "MoELayer", gain_handle: int, wqkv: int, wo: int, x: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                  pos: int, n_heads: int, n_kv: int, head_dim: int, fa: int = 16, fw: int = 24, eps: int = 1, window: int = 0,
                  cos: torch.Tensor | None = None, sin: torch.Tensor | None = None, rope: int = 0, inv_sqrt: int | None = None,
                  pos_dev: torch.Tensor | None = None, ids: torch.Tensor | None = None, gates: torch.Tensor | None = None) -> None:
    """One whole parallel decoder block on the row ``x`` [1, d_model], in place: ``x += attention(h) Wo^T + moe(h)`` with
    ``h = rmsnorm(x, gain)`` (``iie_block_dev``: five launches).  ``ids`` (int32 [k]) / ``gates`` (int64 [k]) receive the routing
    when given.  Raises :class:`NoFusedBlock` for shapes without this form."""
    lib = qk_cuda._lib()
    assert x.is_cuda and x.dtype == torch.int64 and x.is_contiguous()
    assert kcache.dtype == torch.int32 and vcache.dtype == torch.int32 and kcache.is_contiguous() and vcache.is_contiguous()
    if inv_sqrt is None:
        inv_sqrt = int(round((1.0 / head_dim ** 0.5) * (1 << fa)))
    with _CUDA_LOCK:
        rc = lib.iie_block_dev(int(layer.handle), int(gain_handle), int(wqkv), int(wo), x.data_ptr(), kcache.data_ptr(), vcache.data_ptr(),
                               int(pos), pos_dev.data_ptr() if pos_dev is not None else None, int(window or 0),
                               cos.data_ptr() if rope else None, sin.data_ptr() if rope else None, int(rope), n_heads, n_kv, head_dim,
                               int(kcache.shape[1]), int(fa), int(fw), int(eps), int(inv_sqrt),
                               ids.data_ptr() if ids is not None else None, gates.data_ptr() if gates is not None else None, _stream_ptr())
    if rc == 5:
        raise NoFusedBlock("this block shape has no fused form")
    if rc != 0:
        raise CudaContextError(f"decoder block failed with status {rc}")


class DecoderKernel:
    """All blocks of a decoder as one launch per token (``iie_decoder_*``).  ``layers`` = sequence of dicts with ``gain``
    (dense int64 handle), ``moe`` (:class:`MoELayer` with its router), ``wqkv``, ``wo`` (handles), ``k``, ``v`` (int32 CUDA
    caches [n_kv, rows, head_dim]) and ``full`` (bool).  Raises :class:`UnsupportedShape` when the model is outside what the
    one-launch kernel carries; the caller then keeps the per-block entries."""

    class UnsupportedShape(RuntimeError):
        pass

    def __init__(self, layers, n_heads: int, n_kv: int, head_dim: int, window: int, cos: torch.Tensor, sin: torch.Tensor,
                 fa: int = 16, fw: int = 24, eps: int = 1, inv_sqrt: int | None = None):
        lib = qk_cuda._lib()
        rows = int(layers[0]["k"].shape[1])
        if inv_sqrt is None:
            inv_sqrt = int(round((1.0 / head_dim ** 0.5) * (1 << fa)))
        assert cos.is_cuda and sin.is_cuda and cos.dtype == torch.int64 and cos.is_contiguous() and sin.is_contiguous()
        assert cos.shape[0] >= rows and cos.shape[1] == head_dim // 2
        with _CUDA_LOCK:
            self.handle = int(lib.iie_decoder_create(len(layers), n_heads, n_kv, head_dim, int(window or 0), rows, int(fa), int(fw),
                                                     int(eps), int(inv_sqrt), cos.data_ptr(), sin.data_ptr()))
        if self.handle < 0:
            raise self.UnsupportedShape("decoder shape rejected")
        self._keep = (cos, sin, [(L["k"], L["v"]) for L in layers])          # the kernel reads these: keep them alive
        for li, L in enumerate(layers):
            k, v = L["k"], L["v"]
            assert k.dtype == torch.int32 and v.dtype == torch.int32 and k.is_contiguous() and v.is_contiguous()
            assert k.shape == v.shape == (n_kv, rows, head_dim)
            with _CUDA_LOCK:
                rc = lib.iie_decoder_set_layer(self.handle, li, int(L["gain"]), int(L["moe"].handle), int(L["wqkv"]), int(L["wo"]),
                                               k.data_ptr(), v.data_ptr(), 1 if L["full"] else 0)
            if rc != 0:
                self.close()
                if rc == 5:
                    raise self.UnsupportedShape(f"block {li} is outside what the one-launch kernel carries")
                raise CudaContextError(f"decoder block {li} rejected with status {rc}")

    def step(self, x: torch.Tensor, pos_bound: int, pos_dev: torch.Tensor | None = None, ids_out: torch.Tensor | None = None,
             gates_out: torch.Tensor | None = None) -> None:
        """x [1, d_model] int64 updated in place through every block, on the current stream."""
        assert x.is_cuda and x.dtype == torch.int64 and x.is_contiguous()
        with _CUDA_LOCK:
            rc = qk_cuda._lib().iie_decoder_step_dev(self.handle, x.data_ptr(), int(pos_bound),
                                                     pos_dev.data_ptr() if pos_dev is not None else None,
                                                     ids_out.data_ptr() if ids_out is not None else None,
                                                     gates_out.data_ptr() if gates_out is not None else None, _stream_ptr())
        if rc == 5:
            raise self.UnsupportedShape("the visible cache rows exceed what one launch holds")
        if rc != 0:
            raise CudaContextError(f"decoder step failed with status {rc}")

    def close(self) -> None:
        if self.handle >= 0:
            with _CUDA_LOCK:
                qk_cuda._lib().iie_decoder_destroy(self.handle)
            self.handle = -1


def embed(handle: int, token, d_model: int, fa: int = 16, out: torch.Tensor | None = None) -> torch.Tensor:
    """Row ``token`` (an int, or a CUDA int32 tensor holding it) of a registered matrix at 2**fa -> [1, d_model]."""
    lib = qk_cuda._lib()
    if out is None:
        out = torch.empty((1, d_model), dtype=torch.int64, device="cuda")
    on_dev = isinstance(token, torch.Tensor)
    with _CUDA_LOCK:
        rc = lib.iie_embed_dev(int(handle), token.data_ptr() if on_dev else None, 0 if on_dev else int(token), int(fa),
                               out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"embedding look-up failed with status {rc}")
    return out


def argmax(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest value, lowest index on ties -> CUDA int32 tensor [1]."""
    lib = qk_cuda._lib()
    assert x.is_cuda and x.dtype == torch.int64 and x.is_contiguous()
    if out is None:
        out = torch.empty(1, dtype=torch.int32, device=x.device)
    with _CUDA_LOCK:
        rc = lib.iie_argmax_dev(x.data_ptr(), x.numel(), out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"argmax failed with status {rc}")
    return out


def embed_rows(handle: int, tokens: torch.Tensor, d_model: int, fa: int = 16, out: torch.Tensor | None = None) -> torch.Tensor:
    """Rows ``tokens`` (CUDA int32 [B]) of a registered matrix at 2**fa -> [B, d_model], one launch."""
    lib = qk_cuda._lib()
    assert tokens.is_cuda and tokens.dtype == torch.int32 and tokens.is_contiguous()
    B = tokens.numel()
    if out is None:
        out = torch.empty((B, d_model), dtype=torch.int64, device="cuda")
    assert out.is_contiguous() and out.shape == (B, d_model)
    with _CUDA_LOCK:
        rc = lib.iie_embed_rows_dev(int(handle), tokens.data_ptr(), B, int(fa), out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"embedding look-up failed with status {rc}")
    return out


def argmax_rows(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Per row of ``x`` [B, n]: index of the largest value, lowest index on ties -> CUDA int32 [B], one launch."""
    lib = qk_cuda._lib()
    assert x.is_cuda and x.dtype == torch.int64 and x.dim() == 2 and x.is_contiguous()
    if out is None:
        out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    with _CUDA_LOCK:
        rc = lib.iie_argmax_rows_dev(x.data_ptr(), x.shape[0], x.shape[1], out.data_ptr(), _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"argmax failed with status {rc}")
    return out


def workspace_generation() -> int:
    """Changes whenever a scratch buffer of the library is freed (regrown or released).  A CUDA graph captured over the
    device entries holds the addresses of its capture: compare before replaying."""
    return int(qk_cuda.load_library().iie_workspace_generation())


def prefill_launch_counts() -> list:
    """Launches of each tensor-core tile shape since load: [gate/up 3 digits, gate/up 4, Q6_K down 5, Q6_K down 6,
    Q4_K down 5, linear 3, linear 5]."""
    buf = (ctypes.c_uint64 * 8)()
    n = qk_cuda.load_library().iie_prefill_launch_counts(buf, 8)
    return [int(buf[i]) for i in range(n)]


def launch_count() -> int:
    """Kernels launched by the library since it was loaded."""
    return int(qk_cuda.load_library().iie_launch_count())


def set_stage_mask(mask: int) -> None:
    """Profiling: restrict MoELayer.forward to a subset of its stages (0 = all)."""
    with _CUDA_LOCK:
        qk_cuda._lib().iie_profile_stage_mask(int(mask))


def read_flags() -> int:
    """Read and clear the envelope flag word (synchronises): 0 means every result so far is exact."""
    with _CUDA_LOCK:
        return int(qk_cuda._lib().iie_flags_read_clear(_stream_ptr()))


def route(router: int, top_k: int, h: torch.Tensor, fa: int = 16, fw: int = 24):
    """Router logits, top-k expert ids (lowest index wins ties) and sigmoid gates of every row of ``h``.
    ``router`` is a registered matrix with one row per expert.  Returns (ids [T,k] int32, gates [T,k] int64)."""
    lib = qk_cuda._lib()
    assert h.is_cuda and h.dtype == torch.int64 and h.dim() == 2 and h.is_contiguous()
    T = h.shape[0]
    ids = torch.empty((T, top_k), dtype=torch.int32, device=h.device)
    gates = torch.empty((T, top_k), dtype=torch.int64, device=h.device)
    if T == 0:
        return ids, gates
    with _CUDA_LOCK:
        rc = lib.iie_route_dev(int(router), int(top_k), h.data_ptr(), T, int(fa), int(fw), ids.data_ptr(), gates.data_ptr(),
                               _stream_ptr())
    if rc != 0:
        raise CudaContextError(f"routing failed with status {rc}")
    return ids, gates


class MoELayer:
    """One MoE layer with every expert resident on the device.

    ``router`` is a handle (quantised or dense int64), or -1 for an expert shard that is only driven through
    :meth:`experts`; ``gate``, ``up``, ``down`` are sequences of ``n_experts`` handles with uniform quantisation
    type per projection.
    """

    def __init__(self, router: int, gate, up, down, top_k: int, d_model: int, e_ffn: int):
        lib = qk_cuda._lib()
        n = len(gate)
        if len(up) != n or len(down) != n or n <= 0:
            raise ValueError("gate, up and down need the same positive number of handles")
        arr = lambda hs: (ctypes.c_int64 * n)(*[int(v) for v in hs])
        with _CUDA_LOCK:
            self.handle = int(lib.iie_moe_layer_create(int(router), arr(gate), arr(up), arr(down), n, int(top_k),
                                                       int(d_model), int(e_ffn)))
        if self.handle < 0:
            raise CudaContextError("MoE layer creation failed (shape, type or handle mismatch)")
        self.n_experts, self.top_k, self.d_model, self.e_ffn = n, int(top_k), int(d_model), int(e_ffn)

    def forward(self, h: torch.Tensor, fa: int = 16, fw: int = 24, out: torch.Tensor | None = None,
                accumulate: bool = False, want_routes: bool = True):
        """h [T,d_model] int64 -> (out [T,d_model], ids [T,k] int32, gates [T,k] int64).
        Asynchronous on the current stream; call :func:`read_flags` to confirm exactness."""
        lib = qk_cuda._lib()
        h = h.contiguous()
        assert h.is_cuda and h.dtype == torch.int64 and h.dim() == 2 and h.shape[1] == self.d_model
        T = h.shape[0]
        if out is None:
            out = torch.empty((T, self.d_model), dtype=torch.int64, device=h.device)
            accumulate = False
        ids = torch.empty((T, self.top_k), dtype=torch.int32, device=h.device) if want_routes else None
        gates = torch.empty((T, self.top_k), dtype=torch.int64, device=h.device) if want_routes else None
        with _CUDA_LOCK:
            rc = lib.iie_moe_forward_dev(self.handle, h.data_ptr(), T, int(fa), int(fw), int(bool(accumulate)),
                                         out.data_ptr(), ids.data_ptr() if want_routes else None,
                                         gates.data_ptr() if want_routes else None, _stream_ptr())
        if rc != 0:
            raise CudaContextError(f"MoE forward failed with status {rc}")
        return out, ids, gates

    def block(self, x: torch.Tensor, gain_handle: int = -1, fa: int = 16, fw: int = 24, eps: int = 1,
              out: torch.Tensor | None = None, want_routes: bool = True):
        """The block with normalisation and residual: ``moe(x)`` without a gain handle, otherwise
        ``x + moe(rmsnorm(x, gain))``.  ``out`` may be ``x`` itself.  Returns (out, ids, gates)."""
        lib = qk_cuda._lib()
        assert x.is_cuda and x.dtype == torch.int64 and x.dim() == 2 and x.shape[1] == self.d_model and x.is_contiguous()
        T = x.shape[0]
        if out is None:
            out = torch.empty_like(x)
        ids = torch.empty((T, self.top_k), dtype=torch.int32, device=x.device) if want_routes else None
        gates = torch.empty((T, self.top_k), dtype=torch.int64, device=x.device) if want_routes else None
        with _CUDA_LOCK:
            rc = lib.iie_moe_block_dev(self.handle, int(gain_handle), x.data_ptr(), T, int(fa), int(fw), int(eps),
                                       out.data_ptr(), ids.data_ptr() if want_routes else None,
                                       gates.data_ptr() if want_routes else None, _stream_ptr())
        if rc != 0:
            raise CudaContextError(f"MoE block failed with status {rc}")
        return out, ids, gates

    def experts(self, h: torch.Tensor, ids: torch.Tensor, gates: torch.Tensor, expert_base: int = 0, fa: int = 16,
                fw: int = 24, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
        """Expert stage only, with routing supplied by the caller: ``ids`` [T,slots] int32 are expert ids of the
        whole model, this layer owning ``expert_base .. expert_base + n_experts - 1``; other slots are skipped.
        Returns, per row, the sum over this shard's slots of ``floor(down * gate / 2**fa)``."""
        lib = qk_cuda._lib()
        assert h.is_cuda and h.dtype == torch.int64 and h.dim() == 2 and h.shape[1] == self.d_model and h.is_contiguous()
        T = h.shape[0]
        assert ids.dtype == torch.int32 and gates.dtype == torch.int64 and ids.shape == gates.shape and ids.shape[0] == T
        ids, gates = ids.contiguous(), gates.contiguous()
        if out is None:
            out = torch.empty((T, self.d_model), dtype=torch.int64, device=h.device)
            accumulate = False
        if T == 0:
            return out
        with _CUDA_LOCK:
            rc = lib.iie_moe_experts_dev(self.handle, h.data_ptr(), T, ids.data_ptr(), gates.data_ptr(), int(ids.shape[1]),
                                         int(expert_base), int(fa), int(fw), int(bool(accumulate)), out.data_ptr(),
                                         _stream_ptr())
        if rc != 0:
            raise CudaContextError(f"MoE expert stage failed with status {rc}")
        return out

    def close(self):
        if self.handle >= 0:
            with _CUDA_LOCK:
                qk_cuda._lib().iie_moe_layer_destroy(self.handle)
            self.handle = -1
