"""A synthetic 1-bit (Q1_0) decoder of the bonsai shape on one GPU: one whole decode token on the device.

Per layer the sequential residual block of bonsai/src/trinote/infer_int/reference_bonsai.py (941-966 _run_layers,
656-720 _attention_with_cache_bonsai, 603-615 _ffn_ref):

    h = rmsnorm(x, attn_norm);  q, k, v = q1(h, wq), q1(h, wk), q1(h, wv)
    q, k = per-head rmsnorm with a [head_dim] gain, then rotate-half RoPE;  append k, v to the cache
    x += q1(attention(q, cache), wo)
    h = rmsnorm(x, ffn_norm);  x += q1((silu(q1(h, w1)) * q1(h, wu)) >> frac, w2)      # wrapping products

The input row is row `token` of the Q1_0 embedding at 2**frac (q1_rows_fp, 138-146); the head is the Q1_0 output
matrix applied to rmsnorm(x, out_norm) and the greedy pick is the lowest-index arg-max (812-826).

Weights are seeded synthetic sign bits and float16-derived scales; KV caches are seeded int32 values standing in
for a prefill.  Token id and position live in device cells so one captured launch sequence serves every step.
"""
from __future__ import annotations

import numpy as np
import torch

from . import device, q1_gpu
from .model import rope_tables


def synth_q1(out_f: int, nb: int, gen: np.random.Generator, frac: int = 16, smag: float = 0.02):
    """Random Q1_0 tensor: packed sign bytes [out_f, nb, 16] and int32 scales rint(float16(|N(0,1)|*smag) * 2**frac)."""
    bits = gen.integers(0, 256, size=(out_f, nb, 16), dtype=np.uint8)
    sc16 = np.abs(gen.standard_normal((out_f, nb), dtype=np.float32) * smag).astype(np.float16)
    return bits, np.rint(sc16.astype(np.float64) * (1 << frac)).astype(np.int32)


class Q1Decoder:
    """Decoder over given tensors.  ``layers`` yields dicts with int64 gains n1, n2 [d], qn, kn [head_dim], (bits, scale)
    pairs wqkv (Wq, Wk, Wv rows stacked), wo, w1u (gate rows then up rows), w2, and int32 caches k, v
    [n_kv, rows, head_dim] (host arrays or CUDA tensors); ``top`` = dict(embed, head, out_gain)."""

    def __init__(self, d_model: int, n_heads: int, n_kv: int, head_dim: int, d_ffn: int, vocab: int, layers, top, cos, sin,
                 context: int, frac: int = 16):
        self.d, self.H, self.Hkv, self.hd, self.ffn = d_model, n_heads, n_kv, head_dim, d_ffn
        self.vocab, self.frac, self.context = vocab, frac, context
        qd, kd = n_heads * head_dim, n_kv * head_dim
        reg = lambda w: q1_gpu.q1_register_weight(np.ascontiguousarray(w[0]), np.ascontiguousarray(w[1]))
        gain = lambda g: torch.from_numpy(np.ascontiguousarray(g, dtype=np.int64)).cuda()
        dev = lambda c: c if isinstance(c, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(c, dtype=np.int32)).cuda()
        self.layers = []
        for L in layers:
            self.layers.append({"n1": gain(L["n1"]), "n2": gain(L["n2"]), "qn": gain(L["qn"]), "kn": gain(L["kn"]),
                                "wqkv": reg(L["wqkv"]), "wo": reg(L["wo"]), "w1u": reg(L["w1u"]), "w2": reg(L["w2"]),
                                "k": dev(L["k"]), "v": dev(L["v"])})
        self.n_layers = len(self.layers)
        self.embed, self.head, self.out_gain = reg(top["embed"]), reg(top["head"]), gain(top["out_gain"])
        self.cos, self.sin = torch.from_numpy(np.ascontiguousarray(cos)).cuda(), torch.from_numpy(np.ascontiguousarray(sin)).cuda()
        self.pos = torch.tensor([context], dtype=torch.int32, device="cuda")        # position of the next token
        self.token = torch.zeros(1, dtype=torch.int32, device="cuda")               # its id
        z = lambda n: torch.empty((1, n), dtype=torch.int64, device="cuda")
        self.x, self.qkv, self.qkvn, self.att = z(d_model), z(qd + 2 * kd), z(qd + kd), z(qd)
        self.gu, self.logits = z(2 * d_ffn), z(vocab)
        self.rows = int(self.layers[0]["k"].shape[1])
        self._pos_host = int(context)                                               # host mirror of the position cell
        self._graph = None

    def set_position(self, position: int) -> None:
        self.pos.fill_(int(position))
        self._pos_host = int(position)

    def _admit(self, bound: int) -> None:
        """Host-side refusal of a step beyond the bound the launches were sized for or the rows of the cache."""
        if self._pos_host > bound or self._pos_host >= self.rows:
            raise q1_gpu.CudaContextError(
                f"decode step at position {self._pos_host} is beyond the bound {bound} / the {self.rows} cache rows")

    def weight_bytes_per_token(self) -> int:
        """Sign bits + int32 scales every matrix streams for one token (one embedding row excluded)."""
        per_block = 16 + 4
        qd, kd = self.H * self.hd, self.Hkv * self.hd
        rows_in = (qd + 2 * kd) * self.d + self.d * qd + 2 * self.ffn * self.d + self.d * self.ffn
        return (self.n_layers * rows_in + self.vocab * self.d) // 128 * per_block

    def step(self, pos_bound: int) -> None:
        self._admit(pos_bound)
        self._launch_step(pos_bound)
        self._pos_host += 1

    def _launch_step(self, pos_bound: int) -> None:
        """One token: reads ``self.token`` / ``self.pos`` on the device, leaves the next id in ``self.token`` and advances
        ``self.pos``.  Per layer ten launches: norm + digit planes, QKV product, both head norms, attention, planes,
        O product with the residual, norm + planes, gate/up product, SwiGLU + planes, down product with the residual."""
        f, qd, kd = self.frac, self.H * self.hd, self.Hkv * self.hd
        q1_gpu.embed_dev(self.embed, self.token, self.x)
        for L in self.layers:
            q1_gpu.apply_fused_dev(L["wqkv"], self.x, f, self.qkv, norm=True, gain=L["n1"])
            q1_gpu.head_norm_dev(self.qkv, self.H, self.Hkv, self.hd, L["qn"], L["kn"], f, self.qkvn)
            device.attention_decode(self.qkvn[0, :qd], self.qkvn[0, qd:], self.qkv[0, qd + kd:], L["k"], L["v"], pos_bound,
                                    self.H, self.Hkv, self.hd, f, 0, self.cos, self.sin, 2, out=self.att.view(-1), pos_dev=self.pos)
            q1_gpu.apply_fused_dev(L["wo"], self.att, f, self.x, add=self.x)
            q1_gpu.apply_fused_dev(L["w1u"], self.x, f, self.gu, norm=True, gain=L["n2"])
            q1_gpu.apply_fused_dev(L["w2"], self.gu[:, :self.ffn], f, self.x, up=self.gu[:, self.ffn:], add=self.x)
        q1_gpu.apply_fused_dev(self.head, self.x, f, self.logits, norm=True, gain=self.out_gain)
        device.argmax(self.logits.view(-1), out=self.token)
        self.pos += 1

    def capture(self, pos_bound: int) -> None:
        self._admit(pos_bound)
        keep = (self.token.clone(), self.pos.clone())
        self._launch_step(pos_bound)
        torch.cuda.synchronize()
        self._stream = torch.cuda.Stream()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self._stream):
            with torch.cuda.graph(self._graph, stream=self._stream):
                self._launch_step(pos_bound)
        torch.cuda.synchronize()
        self.token.copy_(keep[0]); self.pos.copy_(keep[1])
        self._bound = pos_bound
        self._generation = device.workspace_generation() + q1_gpu.workspace_generation()

    def replay(self) -> None:
        """Replay the captured step; refused on the host past the captured bound or the cache rows, and after the
        library's workspaces were freed or regrown (the graph holds their old addresses)."""
        if self._graph is None:
            raise q1_gpu.CudaContextError("capture() has not been called")
        self._admit(self._bound)
        if device.workspace_generation() + q1_gpu.workspace_generation() != self._generation:
            raise q1_gpu.CudaContextError("library workspaces changed since capture(): the graph must be captured again")
        self._graph.replay()
        self._pos_host += 1

    def decode_token(self, token_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Per-token call with pinned host buffers (int32 [1] in, next id out); needs :meth:`capture` first."""
        self.token.copy_(token_host, non_blocking=True)
        self.replay()
        out_host.copy_(self.token, non_blocking=True)
        torch.cuda.current_stream().synchronize()


class SyntheticQ1Decoder(Q1Decoder):
    """Seeded synthetic tensors of the given shape (defaults: the 8B bonsai shape); ``keep_host`` keeps the host copies
    of every tensor in ``self.host_layers`` / ``self.host_top`` for a CPU checker (small shapes only)."""

    def __init__(self, n_layers: int = 36, d_model: int = 4096, n_heads: int = 32, n_kv: int = 8, head_dim: int = 128,
                 d_ffn: int = 12288, vocab: int = 151936, context: int = 512, max_new: int = 64, rope_base: float = 1e6,
                 seed: int = 1, frac: int = 16, keep_host: bool = False):
        rng = np.random.default_rng(seed)
        rows = context + max_new
        qd, kd = n_heads * head_dim, n_kv * head_dim
        w = lambda out_f, in_f: synth_q1(out_f, in_f // 128, rng, frac)
        gain = lambda n: np.rint((np.abs(rng.standard_normal(n)) + 0.5) * (1 << frac)).astype(np.int64)
        kept = []

        def layers():
            for li in range(n_layers):
                g = torch.Generator(device="cuda").manual_seed(seed * 7919 + li)
                cache = lambda: torch.randint(-(1 << 17), 1 << 17, (n_kv, rows, head_dim), generator=g, device="cuda",
                                              dtype=torch.int32)
                L = {"n1": gain(d_model), "n2": gain(d_model), "qn": gain(head_dim), "kn": gain(head_dim),
                     "wqkv": w(qd + 2 * kd, d_model), "wo": w(d_model, qd), "w1u": w(2 * d_ffn, d_model), "w2": w(d_model, d_ffn),
                     "k": cache(), "v": cache()}
                if keep_host:
                    kept.append(L)
                yield L

        top = {"embed": w(vocab, d_model), "head": w(vocab, d_model), "out_gain": gain(d_model)}
        cos, sin = rope_tables(rows, head_dim, rope_base, frac)
        super().__init__(d_model, n_heads, n_kv, head_dim, d_ffn, vocab, layers(), top, cos, sin, context, frac)
        self.host_layers, self.host_top = (kept, top) if keep_host else (None, None)
