"""A whole synthetic decoder of the 30B-A3B shape on one GPU: the decode step the benchmark times.

Per layer the reference's parallel block (north-mini-code/src/nmc/cohere2.py:357-376 block_cached):

    h = rmsnorm(x, attn_norm);  q, k, v = h Wq^T, h Wk^T, h Wv^T;  rotate q, k on sliding-window layers
    append k, v to the cache;  a = attention(q, cache) Wo^T;  x = x + a + moe(h)

then the tied head (cohere2.py:201-204): logits = rmsnorm(x, output_norm) E^T, greedy pick = arg-max with the
lowest index on ties (engine.py:585), next input = row `token` of E at 2**fa (engine.py:239-243).

Weights are seeded synthetic blocks generated on the device (distributions of ``synth.py``); the KV caches are
filled with seeded int32 values up to the requested context length, standing in for a prefill.  Everything a
step needs stays on the device: the sampled token and the position live in device cells, so one captured
launch sequence serves every step.
"""
from __future__ import annotations

import numpy as np
import torch

from . import device, qk_cuda
from .qk_cuda import Q4_K, Q6_K
from .synth import SyntheticMoEStack, synth_q4k, synth_q6k

SWA_PERIOD = 4          # layers 0, 4, 8, ... attend to everything without rotation; the others use a sliding window + RoPE


def rope_tables(rows: int, head_dim: int, base: float, fa: int):
    """cos/sin at 2**fa, [rows, head_dim//2] (north-mini-code/src/nmc/_bonsai/rope.py:42-66), built on the host
    in float64 exactly as the reference does (round(cos(p * base**(-2i/d)) * 2**fa))."""
    half = head_dim // 2
    inv = np.array([base ** (-(2 * i) / head_dim) for i in range(half)], dtype=np.float64)
    ang = np.arange(rows, dtype=np.float64)[:, None] * inv[None, :]
    return np.rint(np.cos(ang) * (1 << fa)).astype(np.int64), np.rint(np.sin(ang) * (1 << fa)).astype(np.int64)


class SyntheticDecoder:
    def __init__(self, n_layers: int = 48, d_model: int = 2048, n_heads: int = 32, n_kv: int = 4, head_dim: int = 128,
                 e_ffn: int = 768, n_experts: int = 128, top_k: int = 8, vocab: int = 151936, context: int = 4096,
                 max_new: int = 160, window: int = 4096, rope_base: float = 50000.0, seed: int = 1, fa: int = 16, fw: int = 24):
        self.n_layers, self.d, self.H, self.Hkv, self.hd = n_layers, d_model, n_heads, n_kv, head_dim
        self.vocab, self.fa, self.fw, self.window, self.top_k = vocab, fa, fw, window, top_k
        self.rows = context + max_new
        self.moe = SyntheticMoEStack(n_layers, d_model, e_ffn, n_experts, top_k, seed=seed, fa=fa)
        nb = d_model // 256
        self.attn = []
        for li in range(n_layers):
            gen = torch.Generator(device="cuda").manual_seed(seed * 7919 + 1000 + li)
            # Wq, Wk, Wv stacked row-wise into one matrix (rows are independent in the block layout)
            qkv_rows = (n_heads + 2 * n_kv) * head_dim
            wqkv = device.register_weight(synth_q4k(qkv_rows * nb, gen).view(-1), qkv_rows, nb, Q4_K)
            wo = device.register_weight(synth_q4k(d_model * (n_heads * head_dim // 256), gen).view(-1), d_model,
                                        n_heads * head_dim // 256, Q4_K)
            kc = torch.randint(-(1 << 18), 1 << 18, (n_kv, self.rows, head_dim), generator=gen, device="cuda", dtype=torch.int32)
            vc = torch.randint(-(1 << 18), 1 << 18, (n_kv, self.rows, head_dim), generator=gen, device="cuda", dtype=torch.int32)
            self.attn.append({"wqkv": wqkv, "wo": wo, "k": kc, "v": vc})
        gen = torch.Generator(device="cuda").manual_seed(seed * 7919 + 999)
        self.embd = device.register_weight(synth_q6k(vocab * nb, gen).view(-1), vocab, nb, Q6_K)
        gain = torch.round((torch.randn(d_model, generator=gen, device="cuda", dtype=torch.float64).abs() + 0.5)
                           * (1 << fa)).to(torch.int64)
        self.out_gain = gain
        self.out_gain_h = qk_cuda.register_i64(gain.cpu().numpy())
        cos, sin = rope_tables(self.rows, head_dim, rope_base, fa)
        self.cos, self.sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        self.pos = torch.tensor([context], dtype=torch.int32, device="cuda")        # position of the next token
        self.token = torch.zeros(1, dtype=torch.int32, device="cuda")               # its id
        self.context = context
        # scratch rows of a step
        z = lambda n: torch.empty((1, n), dtype=torch.int64, device="cuda")
        self.x, self.hn, self.logits = z(d_model), z(d_model), z(vocab)

    def layer_is_full(self, li: int) -> bool:
        return li % SWA_PERIOD == 0

    def weight_bytes_per_token(self) -> int:
        nb = self.d // 256
        per_layer_attn = (2 * self.H * self.hd + 2 * self.Hkv * self.hd) * nb * 144
        return self.moe.weight_bytes_per_token() + self.n_layers * per_layer_attn + self.vocab * nb * 210

    def kv_bytes_per_token(self, pos: int) -> int:
        total = 0
        for li in range(self.n_layers):
            keys = pos + 1 if self.layer_is_full(li) else min(pos + 1, self.window)
            total += 2 * self.Hkv * keys * self.hd * 4
        return total

    def step(self, pos_bound: int) -> None:
        """One token: reads ``self.token`` / ``self.pos`` on the device, leaves the next token id in ``self.token``
        and advances ``self.pos``.  ``pos_bound`` is a host upper bound of the position (sizes the grids)."""
        fa, fw = self.fa, self.fw
        device.embed(self.embd, self.token, self.d, fa, out=self.x)
        for li in range(self.n_layers):
            a = self.attn[li]
            full = self.layer_is_full(li)
            # MoE half first: it normalises x, leaves the digit planes of h in the library and adds moe(h) to x;
            # the attention half then reads those planes and adds its own term
            self.moe.layers[li].block(self.x, self.moe.gains[li], fa, fw, 1, out=self.x, want_routes=False)
            device.attention_block(a["wqkv"], a["wo"], self.x, a["k"], a["v"], pos_bound, self.H, self.Hkv, self.hd, fa, fw,
                                   0 if full else self.window, self.cos, self.sin, 0 if full else 1, pos_dev=self.pos)
        device.join_block_overlap()                         # no-op unless the halves of a block run side by side
        device.rmsnorm(self.x, self.out_gain_h, fa, 1, out=self.hn)
        device.apply(self.embd, self.hn, self.vocab, fw, out=self.logits)
        device.argmax(self.logits.view(-1), out=self.token)
        self.pos += 1

    def capture(self, pos_bound: int) -> None:
        """Record one step as a CUDA graph valid for every position up to ``pos_bound``; token and position are
        restored afterwards, the KV row written during the warm-up / capture pass is overwritten by the next real step."""
        keep = (self.token.clone(), self.pos.clone())
        self.step(pos_bound)                                   # sizes every workspace
        torch.cuda.synchronize()
        self._stream = torch.cuda.Stream()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self._stream):
            with torch.cuda.graph(self._graph, stream=self._stream):
                self.step(pos_bound)
        torch.cuda.synchronize()
        self.token.copy_(keep[0]); self.pos.copy_(keep[1])
        self._bound = pos_bound

    def replay(self) -> None:
        self._graph.replay()

    def decode_token(self, token_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Public per-token call with host buffers: pinned int32 ``token_host`` [1] in, next id in pinned ``out_host``
        [1]; returns when the id has arrived.  Needs :meth:`capture` first."""
        self.token.copy_(token_host, non_blocking=True)
        self._graph.replay()
        out_host.copy_(self.token, non_blocking=True)
        torch.cuda.current_stream().synchronize()
