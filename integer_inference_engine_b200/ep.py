"""Expert-parallel MoE block: experts sharded over the ranks of a ``torch.distributed`` group.

The reference runs on one device; this is the multi-GPU form of ``Engine._moe``
(north-mini-code/src/nmc/engine.py:375-443).  Rank ``r`` owns experts ``[r*E/P, (r+1)*E/P)`` and its own
slice of the token batch; the router is replicated.  Per block there is one dispatch and one combine exchange:

  1. every rank routes its own rows (top-k ids with lowest-index ties, sigmoid gates);
  2. dispatch: every rank receives every rank's rows with their (id, gate) slots, in fixed-size segments (no size
     negotiation and no host synchronisation, so a decode step stays a fixed launch sequence that one CUDA graph
     can hold); the receiver skips the slots whose expert it does not own;
  3. each rank runs the expert stage of its shard on what it received and produces, per received row, the
     sum over its own experts of ``floor(down * gate / 2**fa)``;
  4. combine: the partial rows of every owner are summed across the ranks and each owner receives its rows.

Why the dispatch is a fixed-size exchange of all rows rather than a packed all-to-all: with top-8 routing over 128
experts a row is needed by every rank with probability > 0.9 at P <= 4 and by 5.3 of 8 ranks on average at P = 8, so
packing would save at most a third of an exchange that is latency-bound (1 MB per block at 64 sequences), at the price
of device-side counts that the host must read before sizing the collective.

Exactness: every per-expert term is floored before any addition and int64 addition wraps associatively and
commutatively, so the sum over ranks is the same bytes in any order and equals the single-device block, whatever the
number of ranks.  ``combine="reduce_scatter"`` lets the collective library add (NCCL: one reduce-scatter, in-switch
where NVLS is available); ``combine="all_to_all"`` moves the partial rows and adds them here in ascending rank order
(any backend, e.g. gloo on CPU).  The dispatch is an all-gather in the first case and an all-to-all of identical
segments in the second.

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
                 group=None, combine: "str | None" = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not split over {self.world} ranks")
        if combine is None:
            combine = "reduce_scatter" if dist.is_initialized() and dist.get_backend(group) == "nccl" else "all_to_all"
        if combine not in ("reduce_scatter", "all_to_all"):
            raise ValueError("combine is 'reduce_scatter' or 'all_to_all'")
        self.combine = combine
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
        # one [T, d + 2k] int64 segment per rank: the rows with their ids and gates side by side
        seg = torch.empty((T, d + 2 * k), dtype=torch.int64, device=x.device)
        seg[:, :d] = x
        seg[:, d:d + k] = ids
        seg[:, d + k:] = gates
        recv = torch.empty((P * T, d + 2 * k), dtype=torch.int64, device=x.device)
        if self.combine == "reduce_scatter":
            dist.all_gather_into_tensor(recv, seg, group=self.group)
        else:
            dist.all_to_all_single(recv, seg.unsqueeze(0).expand(P, T, d + 2 * k).contiguous().view(P * T, d + 2 * k), group=self.group)
        rows = recv[:, :d].contiguous()
        rids = recv[:, d:d + k].to(torch.int32)
        rgates = recv[:, d + k:].contiguous()
        partial = self.experts_fn(rows, rids, rgates, self.expert_base)          # [P*T, d], segment p = rank p's rows
        if self.combine == "reduce_scatter":
            out = torch.empty((T, d), dtype=torch.int64, device=x.device)
            dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=self.group)
        else:
            back = torch.empty_like(partial)
            dist.all_to_all_single(back, partial, group=self.group)              # segment p = rank p's share of my rows
            back = back.view(P, T, d)
            out = back[0].clone()
            for p in range(1, P):                                                # ascending source rank
                out += back[p]
        self.bytes_sent_last = (seg.numel() + partial.numel() // P) * 8 * (P - 1)
        return out, ids, gates


def from_device_layer(router_handle: int, shard, n_experts: int, fa: int = 16, fw: int = 24, group=None,
                      combine: "str | None" = None) -> ExpertParallelMoE:
    """Bind the CUDA entries: ``shard`` is a :class:`integer_inference_engine_b200.device.MoELayer` holding this
    rank's experts (created with ``router=-1``), ``router_handle`` the replicated router with ``n_experts`` rows."""
    from . import device

    def route_fn(x):
        return device.route(router_handle, shard.top_k, x, fa, fw)

    def experts_fn(rows, ids, gates, base):
        return shard.experts(rows, ids, gates, base, fa, fw)

    return ExpertParallelMoE(n_experts, shard.top_k, shard.d_model, route_fn, experts_fn, group, combine)
