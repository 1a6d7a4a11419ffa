"""A whole decoder of the north-mini-code (30B-A3B) shape on one GPU: the decode step the benchmark times.

Per layer the reference's parallel block (north-mini-code/src/nmc/cohere2.py:357-376 block_cached):

    h = rmsnorm(x, attn_norm);  q, k, v = h Wq^T, h Wk^T, h Wv^T;  rotate q, k on sliding-window layers
    append k, v to the cache;  a = attention(q, cache) Wo^T;  x = x + a + moe(h)

then the tied head (cohere2.py:201-204): logits = rmsnorm(x, output_norm) E^T, greedy pick = arg-max with the
lowest index on ties (engine.py:585), next input = row `token` of E at 2**fa (engine.py:239-243).

:class:`Decoder` holds registered weights and int32 KV caches and runs steps; :meth:`Decoder.from_raw` builds one from
raw Q4_K / Q6_K bytes (a checkpoint reader or a test fixture), :class:`SyntheticDecoder` from seeded synthetic blocks
generated on the device (distributions of ``synth.py``) with the caches filled with seeded int32 values up to the
requested context, standing in for a prefill.  Everything a step needs stays on the device: the sampled token and the
position live in device cells, so one captured launch sequence serves every step.
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


class Decoder:
    """Decode steps over registered weights.  ``attn[i]`` = dict(wqkv, wo handles; k, v int32 CUDA caches
    [n_kv, rows, head_dim]); ``moe_layers[i]`` / ``gain_handles[i]`` the MoE layer and the block's norm gain."""

    def __init__(self, *, d_model, n_heads, n_kv, head_dim, top_k, vocab, window, fa, fw, attn, moe_layers, gain_handles,
                 embd, out_gain_h, cos, sin, position, one_launch=False, dense_router=False):
        self.d, self.H, self.Hkv, self.hd = d_model, n_heads, n_kv, head_dim
        self.vocab, self.fa, self.fw, self.window, self.top_k = vocab, fa, fw, window, top_k
        self.attn, self.moe_layers, self.gain_handles = attn, moe_layers, gain_handles
        self.n_layers = len(attn)
        self.embd, self.out_gain_h = embd, out_gain_h
        self.cos, self.sin = cos, sin
        self.rows = int(attn[0]["k"].shape[1])
        self.pos = torch.tensor([position], dtype=torch.int32, device="cuda")       # position of the next token
        self.token = torch.zeros(1, dtype=torch.int32, device="cuda")               # its id
        self._pos_host = int(position)                                              # host mirror of the position cell
        z = lambda n: torch.empty((1, n), dtype=torch.int64, device="cuda")
        self.x, self.hn, self.logits = z(d_model), z(d_model), z(vocab)
        self._graph = None
        self.dense_router = dense_router                 # routers are dense int64 matrices: the blocks run stage by stage
        # a block as five launches (iie_block_dev) where the shape has that form, else as the MoE half followed by the
        # attention half (six launches); settable for comparisons, both give the same bytes
        self.fused_block = not dense_router
        # one_launch: every block inside one persistent kernel where the shape allows it (byte-identical; on B200 it does not
        # yet beat the two entries per block, so it is opt-in)
        self.kernel = None
        if one_launch and not dense_router:
            try:
                self.kernel = device.DecoderKernel(
                    [{"gain": gain_handles[i], "moe": moe_layers[i], "wqkv": attn[i]["wqkv"], "wo": attn[i]["wo"], "k": attn[i]["k"],
                      "v": attn[i]["v"], "full": self.layer_is_full(i)} for i in range(self.n_layers)],
                    n_heads, n_kv, head_dim, window, cos, sin, fa, fw)
            except device.DecoderKernel.UnsupportedShape:
                self.kernel = None

    @classmethod
    def from_raw(cls, layers, embd_raw, out_gain, *, d_model, n_heads, n_kv, head_dim, e_ffn, top_k, vocab, window, rows,
                 rope_base=50000.0, fa=16, fw=24, caches=None, position=0, one_launch=False):
        """``layers[i]`` = dict(gain int64 [d]; wq, wk, wv, wo raw Q4_K bytes; moe=(router, gates, ups, downs) raw Q4_K /
        Q4_K / Q4_K / Q6_K bytes), as a GGUF reader hands them over; ``embd_raw`` the tied Q6_K matrix [vocab, d].
        ``caches[i]`` = (k, v) int64 arrays [n_kv, filled, head_dim] already in the cache (after rotation)."""
        nb = d_model // 256
        attn, moe_layers, gains = [], [], []
        for li, L in enumerate(layers):
            qkv = bytes(L["wq"]) + bytes(L["wk"]) + bytes(L["wv"])                  # rows are independent in the block layout
            wqkv = qk_cuda.register_weight(qkv, (n_heads + 2 * n_kv) * head_dim, nb, Q4_K)
            wo = qk_cuda.register_weight(L["wo"], d_model, n_heads * head_dim // 256, Q4_K)
            kc = torch.zeros((n_kv, rows, head_dim), dtype=torch.int32, device="cuda"); vc = torch.zeros_like(kc)
            if caches is not None:
                k0, v0 = caches[li]
                kc[:, :k0.shape[1]] = torch.from_numpy(np.ascontiguousarray(k0).astype(np.int32)).cuda()
                vc[:, :v0.shape[1]] = torch.from_numpy(np.ascontiguousarray(v0).astype(np.int32)).cuda()
            attn.append({"wqkv": wqkv, "wo": wo, "k": kc, "v": vc})
            router, gate, up, down = L["moe"]
            rh = qk_cuda.register_weight(router, len(gate), nb, Q4_K)
            gh = [qk_cuda.register_weight(w, e_ffn, nb, Q4_K) for w in gate]
            uh = [qk_cuda.register_weight(w, e_ffn, nb, Q4_K) for w in up]
            dh = [qk_cuda.register_weight(w, d_model, e_ffn // 256, Q6_K) for w in down]
            moe_layers.append(device.MoELayer(rh, gh, uh, dh, top_k, d_model, e_ffn))
            gains.append(qk_cuda.register_i64(np.asarray(L["gain"], np.int64)))
        embd = qk_cuda.register_weight(embd_raw, vocab, nb, Q6_K)
        out_gain_h = qk_cuda.register_i64(np.asarray(out_gain, np.int64))
        cos, sin = rope_tables(rows, head_dim, rope_base, fa)
        return cls(d_model=d_model, n_heads=n_heads, n_kv=n_kv, head_dim=head_dim, top_k=top_k, vocab=vocab, window=window,
                   fa=fa, fw=fw, attn=attn, moe_layers=moe_layers, gain_handles=gains, embd=embd, out_gain_h=out_gain_h,
                   cos=torch.from_numpy(cos).cuda(), sin=torch.from_numpy(sin).cuda(), position=position, one_launch=one_launch)

    @classmethod
    def from_gguf(cls, path, rows: "int | None" = None, fa: int = 16, fw: int = 24, one_launch: bool = False):
        """Load a checkpoint of the north-mini-code layout (see :mod:`gguf`; tensor names of
        north-mini-code/src/nmc/engine.py:449-498): Q4_K attention matrices, the dense F32 router as int64 at 2**fw
        (engine.py:245-254), expert tensors split per expert, F32 norm gains at 2**fa, the tied Q6_K embedding / head."""
        from .gguf import ARCH, GGUFFile
        g = GGUFFile(path)
        kv = lambda key: g.kv[f"{ARCH}.{key}"]
        if kv("leading_dense_block_count") != 0:
            raise ValueError("dense leading blocks are not supported by this decoder")
        d, H, Hkv, hd = kv("embedding_length"), kv("attention.head_count"), kv("attention.head_count_kv"), kv("attention.key_length")
        E, k, eff, vocab = kv("expert_count"), kv("expert_used_count"), kv("expert_feed_forward_length"), kv("vocab_size")
        rows = int(rows or kv("context_length"))
        nb = d // 256
        to_fixed = lambda a, frac: np.round(np.asarray(a, np.float64) * (1 << frac)).astype(np.int64)
        attn, moe_layers, gains = [], [], []
        for li in range(kv("block_count")):
            p = f"blk.{li}."
            qkv = g.raw(p + "attn_q.weight") + g.raw(p + "attn_k.weight") + g.raw(p + "attn_v.weight")
            wqkv = qk_cuda.register_weight(qkv, (H + 2 * Hkv) * hd, nb, Q4_K)
            wo = qk_cuda.register_weight(g.raw(p + "attn_output.weight"), d, H * hd // 256, Q4_K)
            kc = torch.zeros((Hkv, rows, hd), dtype=torch.int32, device="cuda")
            attn.append({"wqkv": wqkv, "wo": wo, "k": kc, "v": torch.zeros_like(kc)})
            router = qk_cuda.register_i64(to_fixed(g.f32(p + "ffn_gate_inp.weight"), fw))
            gh = [qk_cuda.register_weight(g.expert(p + "ffn_gate_exps.weight", e), eff, nb, Q4_K) for e in range(E)]
            uh = [qk_cuda.register_weight(g.expert(p + "ffn_up_exps.weight", e), eff, nb, Q4_K) for e in range(E)]
            dh = [qk_cuda.register_weight(g.expert(p + "ffn_down_exps.weight", e), d, eff // 256, Q6_K) for e in range(E)]
            moe_layers.append(device.MoELayer(router, gh, uh, dh, k, d, eff))
            gains.append(qk_cuda.register_i64(to_fixed(g.f32(p + "attn_norm.weight"), fa)))
        embd = qk_cuda.register_weight(g.raw("token_embd.weight"), vocab, nb, Q6_K)
        out_gain_h = qk_cuda.register_i64(to_fixed(g.f32("output_norm.weight"), fa))
        cos, sin = rope_tables(rows, hd, float(kv("rope.freq_base")), fa)
        dec = cls(d_model=d, n_heads=H, n_kv=Hkv, head_dim=hd, top_k=k, vocab=vocab, window=kv("attention.sliding_window"), fa=fa, fw=fw,
                  attn=attn, moe_layers=moe_layers, gain_handles=gains, embd=embd, out_gain_h=out_gain_h,
                  cos=torch.from_numpy(cos).cuda(), sin=torch.from_numpy(sin).cuda(), position=0, one_launch=one_launch,
                  dense_router=True)
        return dec

    def generate(self, prompt, n_new: int):
        """Greedy generation as the reference's ``Engine.generate`` (engine.py:535-597) defines it: the prompt fills the cache
        (here one token at a time, which yields the same cache rows and the same last hidden row as a batched prefill), then
        ``n_new`` tokens are picked, each fed back.  Starts at position 0."""
        self.set_position(0)
        out, picked = [], None
        for i, tok in enumerate(list(prompt)):
            self.token.fill_(int(tok))
            self.step(i)
        picked = int(self.token.item())                        # the pick after the last prompt token is the first new token
        for i in range(int(n_new)):
            out.append(picked)
            if i + 1 == int(n_new):
                break
            self.step(len(prompt) + i)
            picked = int(self.token.item())
        return out

    def layer_is_full(self, li: int) -> bool:
        return li % SWA_PERIOD == 0

    def set_position(self, position: int) -> None:
        self.pos.fill_(int(position))
        self._pos_host = int(position)

    def kv_bytes_per_token(self, pos: int) -> int:
        total = 0
        for li in range(self.n_layers):
            keys = pos + 1 if self.layer_is_full(li) else min(pos + 1, self.window)
            total += 2 * self.Hkv * keys * self.hd * 4
        return total

    def _launch_step(self, pos_bound: int) -> None:
        fa, fw = self.fa, self.fw
        device.embed(self.embd, self.token, self.d, fa, out=self.x)
        done = False
        if self.kernel is not None:
            try:
                self.kernel.step(self.x, pos_bound, self.pos)
                done = True
            except device.DecoderKernel.UnsupportedShape:      # more visible cache rows than one launch holds
                done = False
        for li in range(0 if not done else self.n_layers, self.n_layers):
            a = self.attn[li]
            full = self.layer_is_full(li)
            if self.dense_router:
                # a dense router has no fused routing kernel: norm, products, attention and the MoE stage as separate entries
                qd, kd = self.H * self.hd, self.Hkv * self.hd
                h = device.rmsnorm(self.x, self.gain_handles[li], fa, 1)
                qkv = device.apply(a["wqkv"], h, qd + 2 * kd, fw).view(-1)
                att = device.attention_decode(qkv[:qd], qkv[qd:qd + kd], qkv[qd + kd:], a["k"], a["v"], pos_bound, self.H, self.Hkv,
                                              self.hd, fa, 0 if full else self.window, self.cos, self.sin, 0 if full else 1,
                                              pos_dev=self.pos)
                ao = device.apply(a["wo"], att.view(1, -1), self.d, fw)
                moe, _, _ = self.moe_layers[li].forward(h, fa, fw, want_routes=False)
                self.x += ao
                self.x += moe
                continue
            if self.fused_block:
                # the whole block in five launches (norm + QKV + router rows, attention, O, gate/up, down)
                try:
                    device.decoder_block(self.moe_layers[li], self.gain_handles[li], a["wqkv"], a["wo"], self.x, a["k"], a["v"], pos_bound,
                                         self.H, self.Hkv, self.hd, fa, fw, 1, 0 if full else self.window, self.cos, self.sin,
                                         0 if full else 1, pos_dev=self.pos)
                    continue
                except device.NoFusedBlock:
                    self.fused_block = False
            # MoE half first: it normalises x, leaves the digit planes of h in the library and adds moe(h) to x;
            # the attention half then reads those planes and adds its own term
            self.moe_layers[li].block(self.x, self.gain_handles[li], fa, fw, 1, out=self.x, want_routes=False)
            device.attention_block(a["wqkv"], a["wo"], self.x, a["k"], a["v"], pos_bound, self.H, self.Hkv, self.hd, fa, fw,
                                   0 if full else self.window, self.cos, self.sin, 0 if full else 1, pos_dev=self.pos)
        device.rmsnorm(self.x, self.out_gain_h, fa, 1, out=self.hn)
        device.apply(self.embd, self.hn, self.vocab, fw, out=self.logits)
        device.argmax(self.logits.view(-1), out=self.token)
        self.pos += 1

    def _admit(self, bound: int) -> None:
        """Host-side refusal of a step the launches were not sized for: the position cell must not pass the bound the
        grids cover nor the rows of the cache (the kernels refuse too, but then the step is lost)."""
        if self._pos_host > bound or self._pos_host >= self.rows:
            raise qk_cuda.CudaContextError(
                f"decode step at position {self._pos_host} is beyond the bound {bound} / the {self.rows} cache rows")

    def step(self, pos_bound: int) -> None:
        """One token: reads ``self.token`` / ``self.pos`` on the device, leaves the next token id in ``self.token``
        and advances ``self.pos``.  ``pos_bound`` is a host upper bound of the position (sizes the grids)."""
        self._admit(pos_bound)
        self._launch_step(pos_bound)
        self._pos_host += 1

    def capture(self, pos_bound: int) -> None:
        """Record one step as a CUDA graph valid for every position up to ``pos_bound``; token and position are
        restored afterwards, the KV row written during the warm-up / capture pass is overwritten by the next real step."""
        self._admit(pos_bound)
        keep = (self.token.clone(), self.pos.clone())
        self._launch_step(pos_bound)                           # sizes every workspace
        torch.cuda.synchronize()
        self._stream = torch.cuda.Stream()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self._stream):
            with torch.cuda.graph(self._graph, stream=self._stream):
                self._launch_step(pos_bound)
        torch.cuda.synchronize()
        self.token.copy_(keep[0]); self.pos.copy_(keep[1])
        self._bound = pos_bound
        self._generation = device.workspace_generation()

    def replay(self) -> None:
        """Replay the captured step.  Refused on the host when the position has reached the captured bound or the end of
        the cache, and when the library's workspaces were freed or regrown since the capture (the graph holds their
        old addresses): capture again in either case."""
        if self._graph is None:
            raise qk_cuda.CudaContextError("capture() has not been called")
        self._admit(self._bound)
        if device.workspace_generation() != self._generation:
            raise qk_cuda.CudaContextError("library workspaces changed since capture(): the graph must be captured again")
        self._graph.replay()
        self._pos_host += 1

    def decode_token(self, token_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Public per-token call with host buffers: pinned int32 ``token_host`` [1] in, next id in pinned ``out_host``
        [1]; returns when the id has arrived.  Needs :meth:`capture` first."""
        self.token.copy_(token_host, non_blocking=True)
        self.replay()
        out_host.copy_(self.token, non_blocking=True)
        torch.cuda.current_stream().synchronize()


class SyntheticDecoder(Decoder):
    def __init__(self, n_layers: int = 48, d_model: int = 2048, n_heads: int = 32, n_kv: int = 4, head_dim: int = 128,
                 e_ffn: int = 768, n_experts: int = 128, top_k: int = 8, vocab: int = 151936, context: int = 4096,
                 max_new: int = 160, window: int = 4096, rope_base: float = 50000.0, seed: int = 1, fa: int = 16, fw: int = 24,
                 one_launch: bool = False):
        rows = context + max_new
        self.moe = SyntheticMoEStack(n_layers, d_model, e_ffn, n_experts, top_k, seed=seed, fa=fa)
        nb = d_model // 256
        attn = []
        for li in range(n_layers):
            gen = torch.Generator(device="cuda").manual_seed(seed * 7919 + 1000 + li)
            # Wq, Wk, Wv stacked row-wise into one matrix (rows are independent in the block layout)
            qkv_rows = (n_heads + 2 * n_kv) * head_dim
            wqkv = device.register_weight(synth_q4k(qkv_rows * nb, gen).view(-1), qkv_rows, nb, Q4_K)
            wo = device.register_weight(synth_q4k(d_model * (n_heads * head_dim // 256), gen).view(-1), d_model,
                                        n_heads * head_dim // 256, Q4_K)
            kc = torch.randint(-(1 << 18), 1 << 18, (n_kv, rows, head_dim), generator=gen, device="cuda", dtype=torch.int32)
            vc = torch.randint(-(1 << 18), 1 << 18, (n_kv, rows, head_dim), generator=gen, device="cuda", dtype=torch.int32)
            attn.append({"wqkv": wqkv, "wo": wo, "k": kc, "v": vc})
        gen = torch.Generator(device="cuda").manual_seed(seed * 7919 + 999)
        embd = device.register_weight(synth_q6k(vocab * nb, gen).view(-1), vocab, nb, Q6_K)
        gain = torch.round((torch.randn(d_model, generator=gen, device="cuda", dtype=torch.float64).abs() + 0.5)
                           * (1 << fa)).to(torch.int64)
        self.out_gain = gain
        cos, sin = rope_tables(rows, head_dim, rope_base, fa)
        super().__init__(d_model=d_model, n_heads=n_heads, n_kv=n_kv, head_dim=head_dim, top_k=top_k, vocab=vocab, window=window,
                         fa=fa, fw=fw, attn=attn, moe_layers=self.moe.layers, gain_handles=self.moe.gains, embd=embd,
                         out_gain_h=qk_cuda.register_i64(gain.cpu().numpy()), cos=torch.from_numpy(cos).cuda(),
                         sin=torch.from_numpy(sin).cuda(), position=context, one_launch=one_launch)
        self.context = context

    def weight_bytes_per_token(self) -> int:
        nb = self.d // 256
        per_layer_attn = (2 * self.H * self.hd + 2 * self.Hkv * self.hd) * nb * 144
        return self.moe.weight_bytes_per_token() + self.n_layers * per_layer_attn + self.vocab * nb * 210


def host_view(model: "SyntheticDecoder"):
    """Host copies of everything a CPU checker of a decode step needs, read back from the device: per block the raw
    GGUF-order blocks of Wq / Wk / Wv / Wo, router and experts, the norm gain and the caches (int64), then the tied
    embedding, the output gain and the shape.  For small decoders (it copies every tensor)."""
    from .qk_cuda import Q4_K, Q6_K
    nb = model.d // 256
    layers = []
    for li in range(model.n_layers):
        a, hs = model.attn[li], model.moe.handles[li]
        E = model.moe.n_experts
        qr, kr = model.H * model.hd, model.Hkv * model.hd
        fused = device.export_weight(a["wqkv"], qr + 2 * kr, nb, Q4_K)           # rows of Wq, Wk, Wv stacked
        cut = lambda r0, r1: bytes(fused[r0 * nb * 144:r1 * nb * 144])
        layers.append({
            "gain": hs["gain"].cpu().numpy(), "wq": cut(0, qr), "wk": cut(qr, qr + kr), "wv": cut(qr + kr, qr + 2 * kr),
            "wo": device.export_weight(a["wo"], model.d, qr // 256, Q4_K),
            "k": a["k"].cpu().numpy().astype(np.int64), "v": a["v"].cpu().numpy().astype(np.int64), "full": model.layer_is_full(li),
            "moe": (device.export_weight(hs["router"], E, nb, Q4_K),
                    [device.export_weight(h, model.moe.e_ffn, nb, Q4_K) for h in hs["gate"]],
                    [device.export_weight(h, model.moe.e_ffn, nb, Q4_K) for h in hs["up"]],
                    [device.export_weight(h, model.d, model.moe.e_ffn // 256, Q6_K) for h in hs["down"]])})
    cfg = dict(d=model.d, H=model.H, Hkv=model.Hkv, hd=model.hd, eff=model.moe.e_ffn, E=model.moe.n_experts, k=model.top_k,
               vocab=model.vocab, window=model.window, fa=model.fa, fw=model.fw)
    embd = device.export_weight(model.embd, model.vocab, nb, Q6_K)
    return layers, embd, model.out_gain.cpu().numpy(), cfg
