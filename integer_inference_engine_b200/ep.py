"""Expert-parallel MoE block: experts sharded over the ranks of a ``torch.distributed`` group.

The reference runs on one device; this is the multi-GPU form of ``Engine._moe``
(north-mini-code/src/nmc/engine.py:375-443).  Rank ``r`` owns experts ``[r*E/P, (r+1)*E/P)`` and its own
slice of the token batch; the router is replicated.  Per block there is one dispatch and one combine
exchange, both ``all_to_all_single`` (NCCL on GPUs):

  1. every rank routes its own rows (top-k ids with lowest-index ties, sigmoid gates);
  2. dispatch: a rank sends its rows together with their (id, gate) slots to every other rank, in
     fixed-size segments (one per destination, no size negotiation and no host synchronisation, so a decode
     step stays a fixed launch sequence); the receiver skips the slots whose expert it does not own;
  3. each rank runs the expert stage of its shard on what it received and produces, per received row, the
     sum over its own experts of ``floor(down * gate / 2**fa)``;
  4. combine: those partial rows travel back; the owner adds the P partials in ascending source-rank order.

Exactness: every per-expert term is floored before any addition and int64 addition wraps associatively,
so the result equals the single-device block bit for bit, whatever the number of ranks.

With a group of one rank the same code runs with both exchanges elided.

The two compute steps are injected (``route_fn``, ``experts_fn``) so that the exchange logic can be exercised
on CPU ranks (gloo) with a checker in their place; :func:`from_device_layer` binds the CUDA entries.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


class ExpertParallelMoE:
    def __init__(self, n_experts: int, top_k: int, d_model: int,
                 route_fn: Callable[[torch.Tensor], "tuple[torch.Tensor, torch.Tensor]"],
                 experts_fn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor, int], torch.Tensor],
                 group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not split over {self.world} ranks")
        self.n_experts, self.top_k, self.d_model = int(n_experts), int(top_k), int(d_model)
        self.experts_per_rank = self.n_experts // self.world
        self.expert_base = self.rank * self.experts_per_rank
        self.route_fn, self.experts_fn = route_fn, experts_fn
        self.bytes_sent_last = 0

    def forward(self, x: torch.Tensor):
        """x [T, d_model] int64, the rows this rank owns (every rank must pass the same T).
        Returns (out [T, d_model], ids [T, k] int32, gates [T, k] int64)."""
        T, d, k, P = x.shape[0], self.d_model, self.top_k, self.world
        ids, gates = self.route_fn(x)
        if P == 1:
            self.bytes_sent_last = 0
            return self.experts_fn(x, ids, gates, 0), ids, gates
        # dispatch: one [T, d + 2k] int64 segment per destination (rows, ids, gates side by side)
        seg = torch.empty((T, d + 2 * k), dtype=torch.int64, device=x.device)
        seg[:, :d] = x
        seg[:, d:d + k] = ids
        seg[:, d + k:] = gates
        send = seg.unsqueeze(0).expand(P, T, d + 2 * k).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        recv = recv.view(P * T, d + 2 * k)
        rows = recv[:, :d].contiguous()
        rids = recv[:, d:d + k].to(torch.int32).contiguous()
        rgates = recv[:, d + k:].contiguous()
        partial = self.experts_fn(rows, rids, rgates, self.expert_base)          # [P*T, d], segment p = rank p's rows
        back = torch.empty_like(partial)
        dist.all_to_all_single(back, partial.contiguous(), group=self.group)     # segment p = rank p's share of my rows
        back = back.view(P, T, d)
        out = back[0].clone()
        for p in range(1, P):                                                    # fixed order: ascending source rank
            out += back[p]
        self.bytes_sent_last = (send.numel() + partial.numel()) * 8 * (P - 1) // P
        return out, ids, gates


def from_device_layer(router_handle: int, shard, n_experts: int, fa: int = 16, fw: int = 24, group=None) -> ExpertParallelMoE:
    """Bind the CUDA entries: ``shard`` is a :class:`integer_inference_engine_b200.device.MoELayer` holding this
    rank's experts (created with ``router=-1``), ``router_handle`` the replicated router with ``n_experts`` rows."""
    from . import device

    def route_fn(x):
        return device.route(router_handle, shard.top_k, x, fa, fw)

    def experts_fn(rows, ids, gates, base):
        return shard.experts(rows, ids, gates, base, fa, fw)

    return ExpertParallelMoE(n_experts, shard.top_k, shard.d_model, route_fn, experts_fn, group)
