"""Expert-parallel batched decode of the MoE decoder: ``S`` concurrent sequences over the ranks of a process group.

Partition (the reference runs one sequence on one device; this is the multi-GPU serving form of its decode step,
north-mini-code/src/nmc/cohere2.py:357-383 with the experts of engine.py:375-443 sharded):

* sequences are data-parallel: rank ``r`` owns sequences ``[r*S/P, (r+1)*S/P)`` with their KV caches, and runs norm,
  Q/K/V, rotation, cache append, exact attention, O, routing, head and greedy pick for them;
* experts are sharded: rank ``r`` holds experts ``[r*E/P, (r+1)*E/P)`` of every block; per block one dispatch and one
  combine exchange (:mod:`ep`), NCCL over NVLink on GPUs;
* attention matrices, router, norm gains and the tied embedding / head are replicated.

Every rank draws the replicated tensors from the same seed and its expert shard as a slice of the same seeded model, and
a sequence's cache contents depend only on (seed, block, global sequence index), so the model and its inputs are the same
whatever the number of ranks: the outputs of a sequence must be (and are tested to be) byte-identical for P = 1, 2, 4, 8.

All sequences decode in lockstep at one position.  ``capture()`` records the whole step (every block with its two
collectives) as one CUDA graph.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import device, ep, qk_cuda
from .model import SWA_PERIOD, rope_tables
from .qk_cuda import Q4_K, Q6_K
from .synth import SyntheticMoEStack, synth_q4k, synth_q6k


class ExpertParallelDecoder:
    def __init__(self, n_seqs: int, n_layers: int = 48, d_model: int = 2048, n_heads: int = 32, n_kv: int = 4, head_dim: int = 128,
                 e_ffn: int = 768, n_experts: int = 128, top_k: int = 8, vocab: int = 151936, context: int = 4096, max_new: int = 8,
                 window: int = 4096, rope_base: float = 50000.0, seed: int = 1, fa: int = 16, fw: int = 24, group=None,
                 combine: "str | None" = None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_seqs % self.world or n_experts % self.world:
            raise ValueError(f"{n_seqs} sequences / {n_experts} experts do not split over {self.world} ranks")
        self.S, self.B = n_seqs, n_seqs // self.world
        self.n_layers, self.d, self.H, self.Hkv, self.hd = n_layers, d_model, n_heads, n_kv, head_dim
        self.vocab, self.fa, self.fw, self.window, self.top_k, self.e_ffn = vocab, fa, fw, window, top_k, e_ffn
        self.rows = context + max_new
        self.position = context
        epr = n_experts // self.world
        self.stack = SyntheticMoEStack(n_layers, d_model, e_ffn, n_experts, top_k, seed=seed, fa=fa,
                                       expert_range=(self.rank * epr, (self.rank + 1) * epr) if self.world > 1 else None)
        self.blocks = []
        for li in range(n_layers):
            hs = self.stack.handles[li]
            if self.world > 1:
                self.blocks.append(ep.from_device_layer(hs["router"], self.stack.layers[li], n_experts, fa, fw, group, combine))
            else:
                self.blocks.append(None)                       # one rank: the whole block on the device, nothing to exchange
        nb = d_model // 256
        seq0 = self.rank * self.B
        self.attn = []
        for li in range(n_layers):
            gen = torch.Generator(device="cuda").manual_seed(seed * 7919 + 1000 + li)       # replicated: same on every rank
            qkv_rows = (n_heads + 2 * n_kv) * head_dim
            wqkv = device.register_weight(synth_q4k(qkv_rows * nb, gen).view(-1), qkv_rows, nb, Q4_K)
            wo = device.register_weight(synth_q4k(d_model * (n_heads * head_dim // 256), gen).view(-1), d_model,
                                        n_heads * head_dim // 256, Q4_K)
            kc = torch.empty((self.B, n_kv, self.rows, head_dim), dtype=torch.int32, device="cuda")
            vc = torch.empty_like(kc)
            for b in range(self.B):                            # a sequence's cache depends on its global index only
                g2 = torch.Generator(device="cuda").manual_seed((seed * 104729 + li) * 4099 + seq0 + b)
                kc[b] = torch.randint(-(1 << 18), 1 << 18, (n_kv, self.rows, head_dim), generator=g2, device="cuda", dtype=torch.int32)
                vc[b] = torch.randint(-(1 << 18), 1 << 18, (n_kv, self.rows, head_dim), generator=g2, device="cuda", dtype=torch.int32)
            self.attn.append({"wqkv": wqkv, "wo": wo, "k": kc, "v": vc})
        gen = torch.Generator(device="cuda").manual_seed(seed * 7919 + 999)
        self.embd = device.register_weight(synth_q6k(vocab * nb, gen).view(-1), vocab, nb, Q6_K)
        gain = torch.round((torch.randn(d_model, generator=gen, device="cuda", dtype=torch.float64).abs() + 0.5) * (1 << fa)).to(torch.int64)
        self.out_gain = gain
        self.out_gain_h = qk_cuda.register_i64(gain.cpu().numpy())
        cos, sin = rope_tables(self.rows, head_dim, rope_base, fa)
        self.cos, self.sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        z = lambda *shape: torch.empty(shape, dtype=torch.int64, device="cuda")
        self.x, self.hn, self.logits = z(self.B, d_model), z(self.B, d_model), z(self.B, vocab)
        self.tokens = torch.zeros(self.B, dtype=torch.int32, device="cuda")
        self._graph = None
        self.a2a_bytes_per_block = 0

    def layer_is_full(self, li: int) -> bool:
        return li % SWA_PERIOD == 0

    def blocks_step(self, x: torch.Tensor) -> torch.Tensor:
        """Every block applied to the rows ``x`` [B, d_model] of this rank's sequences, in place, at ``self.position``."""
        fa, fw, qd, kd = self.fa, self.fw, self.H * self.hd, self.Hkv * self.hd
        for li in range(self.n_layers):
            a, full = self.attn[li], self.layer_is_full(li)
            h = device.rmsnorm(x, self.stack.gains[li], fa, 1)
            qkv = device.apply(a["wqkv"], h, qd + 2 * kd, fw)
            att = device.attention_decode_batch(qkv[:, :qd].contiguous(), qkv[:, qd:qd + kd].contiguous(), qkv[:, qd + kd:].contiguous(),
                                                a["k"], a["v"], self.position, self.H, self.Hkv, self.hd, fa, 0 if full else self.window,
                                                self.cos, self.sin, 0 if full else 1)
            ao = device.apply(a["wo"], att, self.d, fw)
            if self.blocks[li] is None:
                moe, _, _ = self.stack.layers[li].forward(h, fa, fw)
            else:
                moe, _, _ = self.blocks[li].forward(h)
                self.a2a_bytes_per_block = self.blocks[li].bytes_sent_last
            x += ao
            x += moe
        return x

    def step(self) -> None:
        """One token for every sequence of this rank: embedding rows of ``self.tokens`` -> blocks -> head -> greedy picks,
        left in ``self.tokens``.  The position does not advance here (see :meth:`advance`)."""
        device.embed_rows(self.embd, self.tokens, self.d, self.fa, out=self.x)
        self.blocks_step(self.x)
        device.rmsnorm(self.x, self.out_gain_h, self.fa, 1, out=self.hn)
        device.apply(self.embd, self.hn, self.vocab, self.fw, out=self.logits)
        device.argmax_rows(self.logits, out=self.tokens)

    def advance(self) -> None:
        if self.position + 1 >= self.rows:
            raise qk_cuda.CudaContextError("the caches are full")
        self.position += 1
        self._graph = None                                   # a captured step is bound to its position

    def capture(self) -> None:
        """Record :meth:`step` at the current position as one CUDA graph (blocks, collectives, head, picks)."""
        keep = self.tokens.clone()
        self.step()                                            # sizes every workspace, warms the collectives up
        torch.cuda.synchronize()
        self._stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self._stream):
            # thread-local capture mode: the collective library's watchdog thread may query events while this thread captures
            with torch.cuda.graph(graph, stream=self._stream, capture_error_mode="thread_local"):
                self.step()
        torch.cuda.synchronize()
        self.tokens.copy_(keep)
        self._graph = graph
        self._generation = device.workspace_generation()

    def replay(self) -> None:
        if self._graph is None:
            raise qk_cuda.CudaContextError("capture() has not been called at this position")
        if device.workspace_generation() != self._generation:
            raise qk_cuda.CudaContextError("library workspaces changed since capture(): the graph must be captured again")
        self._graph.replay()
