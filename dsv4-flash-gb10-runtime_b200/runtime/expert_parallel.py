"""Expert-parallel routed MoE layer: the experts of a layer are split into contiguous ranges, one per GPU
(expert e lives on rank e // (E / world)); tokens are data-parallel.

Per layer and rank:
  1. a token is sent ONCE to every rank that owns at least one of its k experts (at most min(k, world) copies,
     not k): one all-to-all of the row counts, one of the rows, each row carrying the activation (bf16 [K]), the
     token's k global expert ids and its k router weights;
  2. the owner masks the ids that are not its own (negative id = skip) and runs the batched tensor-core layer
     (moe_batched.moe_forward) over the rows it received: one partial output row per (token, rank), already
     weighted and summed over that rank's experts;
  3. the partial rows travel back with the mirrored all-to-all;
  4. every token adds its partial rows in rank order in FP32 (fixed order: deterministic) and rounds to bf16.

The collectives are torch.distributed all_to_all_single calls (NCCL on GPUs, gloo in the CPU tests); received
rows land in this rank's own memory before any kernel reads them.  One host synchronisation per layer (the split
sizes of the variable all-to-all).  The reference has no multi-GPU path at all; the contract is that the result
equals the single-GPU layer on the same inputs up to the bf16 rounding of the partial rows.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.distributed as dist


def dispatch_mask(ids: torch.Tensor, experts_per_rank: int, world: int) -> torch.Tensor:
    """bool [world, T]: which token goes to which rank (a token at most once per rank)."""
    T = ids.shape[0]
    dest = torch.div(ids.to(torch.int64), experts_per_rank, rounding_mode="floor")
    mask = torch.zeros(T, world, dtype=torch.bool, device=ids.device)
    mask.scatter_(1, dest.clamp_(0, world - 1), True)
    return mask.t().contiguous()


def plan_dispatch(ids: torch.Tensor, experts_per_rank: int, world: int):
    """Which token goes to which rank.

    Returns (token_of, send_counts): `token_of` lists token indices grouped by destination rank (ranks ascending,
    tokens ascending inside a rank, a token at most once per rank); `send_counts[r]` rows go to rank r.
    """
    mask = dispatch_mask(ids, experts_per_rank, world)
    return mask.nonzero()[:, 1].contiguous(), mask.sum(dim=1)


def _all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


def ep_moe_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, n_experts: int,
                   local_forward: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                   group: Optional[dist.ProcessGroup] = None, out_dim: Optional[int] = None) -> torch.Tensor:
    """x [T, K] (this rank's tokens), ids int32 [T, k] GLOBAL expert ids, weights float32 [T, k].

    `local_forward(rows [R, K], local_ids int32 [R, k], w float32 [R, k]) -> [R, O]` runs this rank's experts on
    the rows (on a GPU: moe_forward bound to the local bank); local_ids are indices into the local bank, -1 where
    the expert belongs to another rank.  `out_dim` is O (default: K).  Returns [T, O] in x's dtype.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    per = n_experts // world
    T, k = ids.shape
    K = x.shape[1]
    O = K if out_dim is None else int(out_dim)
    mask = dispatch_mask(ids, per, world)                             # [world, T]
    counts_out = mask.sum(dim=1).to(torch.int64)
    counts_in = torch.empty(world, dtype=torch.int64, device=x.device)
    dist.all_to_all_single(counts_in, counts_out, group=group)
    both = torch.stack([counts_out, counts_in]).tolist()              # the layer's one host synchronisation
    send_l, recv_l = [int(c) for c in both[0]], [int(c) for c in both[1]]
    # positions of the set entries of the mask in (rank, token) order; the count is known on the host by now, so no
    # second synchronisation (a stable sort of the flags instead of nonzero())
    flat = mask.reshape(-1)
    order = torch.sort(flat.to(torch.uint8), descending=True, stable=True).indices[: sum(send_l)]
    token_of = order % T

    # one payload row per (token, destination): activation | k ids | k weights, as bytes
    xb = x.contiguous().view(torch.uint8).view(T, -1)
    ib = ids.to(torch.int32).contiguous().view(torch.uint8).view(T, -1)
    wb = weights.to(torch.float32).contiguous().view(torch.uint8).view(T, -1)
    payload = torch.cat([xb, ib, wb], dim=1)[token_of]
    got = _all_to_all_rows(payload, send_l, recv_l, group)
    nx, ni = xb.shape[1], ib.shape[1]
    rows = got[:, :nx].contiguous().view(x.dtype).view(-1, K)
    gids = got[:, nx:nx + ni].contiguous().view(torch.int32).view(-1, k)
    wts = got[:, nx + ni:].contiguous().view(torch.float32).view(-1, k)
    local = gids - rank * per
    local = torch.where((local >= 0) & (local < per), local, torch.full_like(local, -1))

    if rows.shape[0] > 0:
        y = local_forward(rows, local.contiguous(), wts)
    else:
        y = rows.new_empty((0, O))
    back = _all_to_all_rows(y, recv_l, send_l, group)                 # partial rows return in `token_of` order
    acc = torch.zeros(T, O, dtype=torch.float32, device=x.device)
    start = 0
    for n in send_l:                                                  # rank order; a token at most once per rank
        if n:
            acc.index_add_(0, token_of[start:start + n], back[start:start + n].float())
        start += n
    return acc.to(x.dtype)


def ep_moe_forward_gathered(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, n_experts: int,
                            local_forward: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                            group: Optional[dist.ProcessGroup] = None, out_dim: Optional[int] = None) -> torch.Tensor:
    """The same layer for the case that EVERY rank holds the same number of tokens T, without any data-dependent
    shape: all-gather of the tokens (activation, ids, weights), every rank runs its own experts over all world * T
    tokens with the ids of other ranks masked (-1), and a reduce-scatter (FP32 sum) brings every token's partial
    rows home.  No host synchronisation, no sorting or gathering, two collectives whose sizes do not depend on the
    routing (so the whole layer can be captured in a CUDA graph); the price is wire volume (every token visits
    every rank) and that the summation order over ranks is the collective's (fixed for a given communicator, but
    not "rank order" as in ep_moe_forward).  On a backend without reduce-scatter (gloo) an all-reduce is used.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    per = n_experts // world
    T, k = ids.shape
    K = x.shape[1]
    O = K if out_dim is None else int(out_dim)
    xg = torch.empty(world * T, K, dtype=x.dtype, device=x.device)
    ig = torch.empty(world * T, k, dtype=torch.int32, device=x.device)
    wg = torch.empty(world * T, k, dtype=torch.float32, device=x.device)
    for dst, src in ((xg, x), (ig, ids.to(torch.int32)), (wg, weights.to(torch.float32))):
        try:
            dist.all_gather_into_tensor(dst, src.contiguous(), group=group)
        except (RuntimeError, NotImplementedError):
            parts = [torch.empty_like(src) for _ in range(world)]
            dist.all_gather(parts, src.contiguous(), group=group)
            dst.copy_(torch.cat(parts, dim=0))
    local = ig - rank * per
    local = torch.where((local >= 0) & (local < per), local, torch.full_like(local, -1))
    y = local_forward(xg, local, wg).float()                          # [world * T, O]; zero rows where nothing is local
    out = torch.empty(T, O, dtype=torch.float32, device=x.device)
    try:
        dist.reduce_scatter_tensor(out, y, op=dist.ReduceOp.SUM, group=group)
    except (RuntimeError, NotImplementedError):
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        out = y[rank * T:(rank + 1) * T]
    return out.to(x.dtype)


class PeerCombine:
    """Receive buffers in symmetric memory for ep_moe_forward_peer: two buffers of bf16 [world, T, O] per rank
    (alternating between calls, so one barrier per call suffices), mapped on every rank of the group."""

    def __init__(self, tokens_per_rank: int, out_dim: int, device, group: Optional[dist.ProcessGroup] = None,
                 in_dim: Optional[int] = None, k: Optional[int] = None):
        """With in_dim (K) and k given, the context also holds this rank's PUBLISHED inputs in symmetric memory
        (x bf16 [T, K], ids int32 [T, k], weights float32 [T, k]) for ep_moe_forward_peer_inputs."""
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.T, self.O = int(tokens_per_rank), int(out_dim)
        self.K, self.k = in_dim, k
        if in_dim is not None and k is not None:
            import ctypes as _ct
            nx, nm = self.T * in_dim * 2, self.T * k * 4
            nx_al = (nx + 255) & ~255
            nm_al = (nm + 255) & ~255
            self.pub = symm_mem.empty(nx_al + 2 * nm_al, dtype=torch.uint8, device=device)
            self.pub_handle = symm_mem.rendezvous(self.pub, group)
            self.pub_x = self.pub[:nx].view(torch.bfloat16).view(self.T, in_dim)
            self.pub_ids = self.pub[nx_al:nx_al + nm].view(torch.int32).view(self.T, k)
            self.pub_w = self.pub[nx_al + nm_al:nx_al + nm_al + nm].view(torch.float32).view(self.T, k)
            self._x_ptrs = (_ct.c_void_p * self.world)()
            self._ids_ptrs = (_ct.c_void_p * self.world)()
            self._w_ptrs = (_ct.c_void_p * self.world)()
            for r in range(self.world):
                base = int(self.pub_handle.buffer_ptrs[r])
                self._x_ptrs[r], self._ids_ptrs[r], self._w_ptrs[r] = base, base + nx_al, base + nx_al + nm_al
        self.slab = self.world * self.T * self.O
        self.buf = symm_mem.empty(2 * self.slab, dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.calls = 0
        import ctypes
        self._ptr_arrays = []
        for half in range(2):
            arr = (ctypes.c_void_p * self.world)()
            for r in range(self.world):
                arr[r] = int(self.handle.buffer_ptrs[r]) + half * self.slab * 2
            self._ptr_arrays.append(arr)

    def next_half(self) -> int:
        half = self.calls & 1
        self.calls += 1
        return half


def ep_moe_forward_peer(ctx: PeerCombine, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, n_experts: int,
                        local_bank: Dict[str, torch.Tensor], group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """ep_moe_forward_gathered with the return path fused into the layer: after the all-gather of the tokens every
    rank runs its experts over all tokens, and the layer's combine kernel stores each token's partial row straight
    into the home rank's receive buffer (peer memory over NVLink: the exchange is the kernel's epilogue, there is no
    reduce-scatter); one barrier over the ranks, then every rank adds the `world` partial rows of its tokens in rank
    order (deterministic).  Every rank must hold ctx.T tokens.  No host synchronisation."""
    from ctypes import c_int
    from . import _capi
    from .moe_batched import forward_workspace_bytes
    lib = _capi.load("moe")
    world, rank = ctx.world, ctx.rank
    per = n_experts // world
    T, k = ids.shape
    K = x.shape[1]
    if T != ctx.T or n_experts % world:
        raise ValueError("ep_moe_forward_peer: every rank must hold ctx.T tokens and the experts must split evenly")
    xg = torch.empty(world * T, K, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(xg, x.contiguous(), group=group)
    # ids and weights travel together (one collective): [T, 2k] 32-bit words per rank
    ids32 = ids.to(torch.int32).contiguous()
    meta = torch.cat([ids32, weights.to(torch.float32).contiguous().view(torch.int32)], dim=1)
    mg = torch.empty(world * T, 2 * k, dtype=torch.int32, device=x.device)
    dist.all_gather_into_tensor(mg, meta, group=group)
    ig = mg[:, :k]
    wg = mg[:, k:].contiguous().view(torch.float32)
    local = ig - rank * per
    local = torch.where((local >= 0) & (local < per), local, torch.full_like(local, -1)).contiguous()
    E_local, hidden, out_dim = local_bank["w1p"].shape[0], local_bank["w1p"].shape[1], local_bank["w2p"].shape[1]
    if out_dim != ctx.O:
        raise ValueError("ep_moe_forward_peer: out_dim differs from the context's")
    ws = torch.empty(forward_workspace_bytes(world * T, k, K, hidden, out_dim, E_local), dtype=torch.uint8, device=x.device)
    half = ctx.next_half()
    rc = lib.mxfp4_moe_forward_ep(_capi.ptr(xg), _capi.ptr(local_bank["w1p"]), _capi.ptr(local_bank["w3p"]),
                                  _capi.ptr(local_bank["w2p"]), _capi.ptr(local_bank["w1s"]), _capi.ptr(local_bank["w3s"]),
                                  _capi.ptr(local_bank["w2s"]), _capi.ptr(local), _capi.ptr(wg), c_int(world * T),
                                  c_int(E_local), c_int(K), c_int(hidden), c_int(out_dim), c_int(k),
                                  ctx._ptr_arrays[half], c_int(world), c_int(rank), c_int(T), _capi.ptr(ws),
                                  _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_forward_ep returned {rc}")
    ctx.handle.barrier()                                             # every rank's partial rows have landed
    out = torch.empty(T, out_dim, dtype=torch.bfloat16, device=x.device)
    mine = ctx.buf[half * ctx.slab:(half + 1) * ctx.slab]
    rc = lib.mxfp4_moe_ep_sum(_capi.ptr(mine), _capi.ptr(ids32), c_int(k), c_int(per), c_int(world), c_int(T),
                              c_int(out_dim), _capi.ptr(out), _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_ep_sum returned {rc}")
    return out


def ep_moe_forward_peer_inputs(ctx: PeerCombine, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                               n_experts: int, local_bank: Dict[str, torch.Tensor],
                               marks: Optional[list] = None) -> torch.Tensor:
    """ep_moe_forward_peer without any collective library on the path: every rank copies its tokens (activations,
    ids, weights) into its published symmetric-memory buffers; after a barrier every rank runs its experts over the
    whole batch, READING each token from the rank that published it (the quantiser and a small id kernel load over
    NVLink) and storing each partial row into the home rank's receive buffer; a second barrier, then the rank-order
    sum.  The context must have been built with in_dim and k.  Block-scaled tensor-core path only.
    `marks`: a list that receives (name, CUDA event) pairs after every step of the call (diagnostic timing)."""
    from ctypes import c_int

    def mark(name):
        if marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    from . import _capi
    lib = _capi.load("moe")
    world, rank = ctx.world, ctx.rank
    per = n_experts // world
    T, k = ids.shape
    K = x.shape[1]
    if ctx.K != K or ctx.k != k or T != ctx.T or n_experts % world:
        raise ValueError("ep_moe_forward_peer_inputs: shapes differ from the context's")
    E_local, hidden, out_dim = local_bank["w1p"].shape[0], local_bank["w1p"].shape[1], local_bank["w2p"].shape[1]
    if out_dim != ctx.O or E_local != per:
        raise ValueError("ep_moe_forward_peer_inputs: bank does not match the context")
    mark("start")
    # a caller whose producer wrote straight into the published buffers (ctx.pub_x / pub_ids / pub_w) has nothing to copy
    if x.data_ptr() != ctx.pub_x.data_ptr():
        ctx.pub_x.copy_(x)
    if ids.data_ptr() != ctx.pub_ids.data_ptr():
        ctx.pub_ids.copy_(ids)
    if weights.data_ptr() != ctx.pub_w.data_ptr():
        ctx.pub_w.copy_(weights)
    mark("publish")
    ctx.handle.barrier()                                             # every rank's tokens are published
    mark("barrier_published")
    need = int(lib.mxfp4_moe_forward_ep2_workspace_bytes(c_int(world), c_int(T), c_int(k), c_int(K), c_int(hidden),
                                                         c_int(out_dim), c_int(E_local)))
    ws = getattr(ctx, "_layer_ws", None)
    if ws is None or ws.numel() < need:
        ws = ctx._layer_ws = torch.empty(need, dtype=torch.uint8, device=x.device)
    half = ctx.next_half()
    rc = lib.mxfp4_moe_forward_ep2(ctx._x_ptrs, ctx._ids_ptrs, ctx._w_ptrs, _capi.ptr(local_bank["w1p"]),
                                   _capi.ptr(local_bank["w3p"]), _capi.ptr(local_bank["w2p"]), _capi.ptr(local_bank["w1s"]),
                                   _capi.ptr(local_bank["w3s"]), _capi.ptr(local_bank["w2s"]), c_int(T), c_int(E_local),
                                   c_int(K), c_int(hidden), c_int(out_dim), c_int(k), ctx._ptr_arrays[half], c_int(world),
                                   c_int(rank), _capi.ptr(ws), _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_forward_ep2 returned {rc}")
    mark("layer")
    ctx.handle.barrier()                                             # every rank's partial rows have landed
    mark("barrier_rows_landed")
    out = torch.empty(T, out_dim, dtype=torch.bfloat16, device=x.device)
    mine = ctx.buf[half * ctx.slab:(half + 1) * ctx.slab]
    rc = lib.mxfp4_moe_ep_sum(_capi.ptr(mine), _capi.ptr(ctx.pub_ids), c_int(k), c_int(per), c_int(world), c_int(T),
                              c_int(out_dim), _capi.ptr(out), _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_ep_sum returned {rc}")
    mark("sum")
    return out


def shard_bank(bank: Dict[str, torch.Tensor], rank: int, world: int) -> Dict[str, torch.Tensor]:
    """This rank's contiguous range of experts of a bank stacked over all experts."""
    n = bank["w1p"].shape[0]
    per = n // world
    return {name: t[rank * per:(rank + 1) * per].contiguous() for name, t in bank.items()}


__all__ = ["dispatch_mask", "plan_dispatch", "ep_moe_forward", "ep_moe_forward_gathered", "PeerCombine",
           "ep_moe_forward_peer", "ep_moe_forward_peer_inputs", "shard_bank"]
