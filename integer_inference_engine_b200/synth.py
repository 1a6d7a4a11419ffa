"""Seeded synthetic tensors generated directly on the device, with the benchmark's distributions.

Q4_K: d, dmin = float16(|N(0,1)| * 0.01), 12 scale bytes and 128 nibble bytes uniform.
Q6_K: ql, qh uniform bytes, int8 scales uniform over [-128,127], d = float16(|N(0,1)| * 0.01).
Any byte pattern is a valid block, so the tensors are drawn as raw bytes and the fp16 fields are
overwritten.  The raw tensors only live until they are registered (the library keeps its own copy).
"""
from __future__ import annotations

import torch

from . import device
from .qk_cuda import Q4_K, Q6_K


def _halves(n: int, mag: float, gen: torch.Generator) -> torch.Tensor:
    v = (torch.randn(n, generator=gen, device="cuda", dtype=torch.float32).abs() * mag).to(torch.float16)
    return v.view(torch.uint8).view(n, 2)


def synth_q4k(n_blocks_total: int, gen: torch.Generator, dmag: float = 0.01) -> torch.Tensor:
    raw = torch.randint(0, 256, (n_blocks_total, 144), dtype=torch.uint8, device="cuda", generator=gen)
    raw[:, 0:2] = _halves(n_blocks_total, dmag, gen)
    raw[:, 2:4] = _halves(n_blocks_total, dmag, gen)
    return raw


def synth_q6k(n_blocks_total: int, gen: torch.Generator, dmag: float = 0.01) -> torch.Tensor:
    raw = torch.randint(0, 256, (n_blocks_total, 210), dtype=torch.uint8, device="cuda", generator=gen)
    raw[:, 208:210] = _halves(n_blocks_total, dmag, gen)
    return raw


class SyntheticMoEStack:
    """``n_layers`` MoE blocks of the 30B-A3B shape: per layer an int64 RMSNorm gain
    (to_fixed(|N(0,1)| + 0.5)), a Q4_K router [E,d], and E experts with Q4_K gate/up [eff,d] and
    Q6_K down [d,eff].  All experts stay resident.

    ``expert_range=(lo, hi)`` keeps only experts lo..hi-1 (an expert-parallel shard): the tensors are drawn
    exactly as for the full stack, so every shard of the same seed is a slice of the same model; the layers
    are then router-less shards and the replicated router handles are in ``handles[i]["router"]``."""

    def __init__(self, n_layers: int, d_model: int = 2048, e_ffn: int = 768, n_experts: int = 128, top_k: int = 8,
                 seed: int = 1, fa: int = 16, expert_range: "tuple[int, int] | None" = None):
        from . import qk_cuda
        lo, hi = expert_range if expert_range is not None else (0, n_experts)
        self.expert_range = (lo, hi)
        self.n_layers, self.d_model, self.e_ffn, self.n_experts, self.top_k, self.fa = \
            n_layers, d_model, e_ffn, n_experts, top_k, fa
        nb_in, nb_dn = d_model // 256, e_ffn // 256
        self.layers, self.gains, self.handles = [], [], []
        for li in range(n_layers):
            gen = torch.Generator(device="cuda").manual_seed(seed * 100003 + li)
            gain = torch.round((torch.randn(d_model, generator=gen, device="cuda", dtype=torch.float64).abs() + 0.5)
                               * (1 << fa)).to(torch.int64)
            gain_h = qk_cuda.register_i64(gain.cpu().numpy())
            router = synth_q4k(n_experts * nb_in, gen)
            router_h = device.register_weight(router.view(-1), n_experts, nb_in, Q4_K)
            gate = synth_q4k(n_experts * e_ffn * nb_in, gen).view(n_experts, -1)
            up = synth_q4k(n_experts * e_ffn * nb_in, gen).view(n_experts, -1)
            down = synth_q6k(n_experts * d_model * nb_dn, gen).view(n_experts, -1)
            gh = [device.register_weight(gate[e], e_ffn, nb_in, Q4_K) for e in range(lo, hi)]
            uh = [device.register_weight(up[e], e_ffn, nb_in, Q4_K) for e in range(lo, hi)]
            dh = [device.register_weight(down[e], d_model, nb_dn, Q6_K) for e in range(lo, hi)]
            del router, gate, up, down
            self.layers.append(device.MoELayer(router_h if expert_range is None else -1, gh, uh, dh, top_k, d_model, e_ffn))
            self.gains.append(gain_h)
            self.handles.append({"router": router_h, "gate": gh, "up": uh, "down": dh, "gain": gain, "gain_h": gain_h})

    # bytes of weights one decoded token touches: per layer the router and top_k whole experts
    def weight_bytes_per_token(self) -> int:
        nb_in, nb_dn = self.d_model // 256, self.e_ffn // 256
        expert = 2 * self.e_ffn * nb_in * 144 + self.d_model * nb_dn * 210
        return self.n_layers * (self.n_experts * nb_in * 144 + self.top_k * expert)

    def decode_step(self, x: torch.Tensor, fw: int = 24) -> torch.Tensor:
        """x [T,d] int64, updated in place through every block: x += moe(rmsnorm(x, gain))."""
        for layer, gain_h in zip(self.layers, self.gains):
            layer.block(x, gain_h, self.fa, fw, 1, out=x, want_routes=False)
        return x
