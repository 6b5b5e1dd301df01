"""Expert-parallel routed MoE layer: the experts of a layer are split into contiguous ranges, one per GPU
(expert e lives on rank e // (E / world)); tokens are data-parallel.

Per layer and rank:
  1. every (token, expert) pair is sent to the rank that owns the expert: one all-to-all of the pair counts,
     one of the activation rows (bf16 [pairs, K]) with their local expert index and router weight;
  2. the owner runs the batched tensor-core layer (moe_batched.moe_forward) over the rows it received, each row
     being a one-expert token, and gets one weighted output row per pair;
  3. the output rows travel back with the mirrored all-to-all;
  4. every token sums its k rows in the router's order (fixed order: deterministic).

The collectives are torch.distributed all_to_all_single calls (NCCL on GPUs, gloo in the CPU tests); received
rows land in this rank's own memory before any kernel reads them.  The reference has no multi-GPU path at all;
the contract is that the result equals the single-GPU layer on the same inputs.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.distributed as dist


def plan_dispatch(ids: torch.Tensor, experts_per_rank: int, world: int):
    """Sort the T*k pairs by destination rank.

    Returns (order, send_counts, local_expert): `order` lists pair indices (t * k + j) grouped by destination rank,
    stable inside a rank; `send_counts[r]` pairs go to rank r; `local_expert` is the expert's index on its owner,
    in `order`.
    """
    flat = ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=world)[:world]
    local_expert = (flat - dest * experts_per_rank)[order].to(torch.int32)
    return order, send_counts, local_expert


def _all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


def ep_moe_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, n_experts: int,
                   local_forward: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                   group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """x [T, K] (this rank's tokens), ids int32 [T, k] GLOBAL expert ids, weights float32 [T, k].

    `local_forward(rows [R, K], local_ids int32 [R, 1], w float32 [R, 1]) -> [R, O]` runs this rank's experts
    (on a GPU: moe_forward bound to the local bank).  Returns [T, O] in x's dtype.
    """
    world = dist.get_world_size(group)
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    T, k = ids.shape
    order, send_counts, local_expert = plan_dispatch(ids, n_experts // world, world)
    send_counts_l = [int(c) for c in send_counts.tolist()]
    counts_in = torch.empty(world, dtype=torch.int64, device=x.device)
    dist.all_to_all_single(counts_in, send_counts.to(torch.int64).to(x.device), group=group)
    recv_counts_l = [int(c) for c in counts_in.tolist()]

    token_of = torch.div(order, k, rounding_mode="floor")
    rows = _all_to_all_rows(x[token_of], send_counts_l, recv_counts_l, group)
    loc = _all_to_all_rows(local_expert.to(x.device).unsqueeze(1), send_counts_l, recv_counts_l, group)
    w_sorted = weights.reshape(-1)[order].unsqueeze(1)
    wts = _all_to_all_rows(w_sorted, send_counts_l, recv_counts_l, group)

    if rows.shape[0] > 0:
        y = local_forward(rows, loc.contiguous(), wts.contiguous())
    else:
        y = rows.new_empty((0, 0))
    out_dim = torch.tensor([y.shape[1] if y.numel() else 0], dtype=torch.int64, device=x.device)
    dist.all_reduce(out_dim, op=dist.ReduceOp.MAX, group=group)      # a rank without rows learns the width
    O = int(out_dim.item())
    if y.numel() == 0:
        y = rows.new_empty((0, O))
    back = _all_to_all_rows(y, recv_counts_l, send_counts_l, group)   # rows return in `order`
    per_pair = torch.empty((T * k, O), dtype=back.dtype, device=x.device)
    per_pair[order] = back
    return per_pair.view(T, k, O).float().sum(dim=1).to(x.dtype)       # j = 0 .. k-1: fixed order


def shard_bank(bank: Dict[str, torch.Tensor], rank: int, world: int) -> Dict[str, torch.Tensor]:
    """This rank's contiguous range of experts of a bank stacked over all experts."""
    n = bank["w1p"].shape[0]
    per = n // world
    return {name: t[rank * per:(rank + 1) * per].contiguous() for name, t in bank.items()}


__all__ = ["plan_dispatch", "ep_moe_forward", "shard_bank"]
