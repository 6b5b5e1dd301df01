"""Expert-parallel dispatch / combine bookkeeping on CPU ranks (gloo, world size 2 and 4): with a stand-in for the
local expert computation the distributed result must equal the single-process one exactly."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_expert(rows, expert_global, w):
    # stands for FFN_e(x) * w: distinguishes experts and keeps the row content
    return rows.float() * (expert_global.float() + 1.0) * w


def _fake_layer(rows, global_ids, w, lo, hi):
    """Weighted sum over the experts lo <= id < hi of every row, rounded to the row dtype (what one rank returns)."""
    acc = torch.zeros(rows.shape[0], rows.shape[1])
    for j in range(global_ids.shape[1]):
        e = global_ids[:, j:j + 1]
        mine = (e >= lo) & (e < hi)
        acc += torch.where(mine, _fake_expert(rows, e, w[:, j:j + 1]), torch.zeros(()))
    return acc.to(rows.dtype)


def _worker(rank, world, port, T, E, k, K):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as entry
    entry.load_package()
    ep = importlib.import_module("dsv4_b200.runtime.expert_parallel")
    g = torch.Generator().manual_seed(100 + rank)                     # every rank has its own tokens
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    ids = torch.rand(T, E, generator=g).topk(k).indices.to(torch.int32)
    if rank == 0:
        ids[:, 0] = 0                                                  # skew: rank 0's tokens all hit expert 0
        ids[:, 1:] = torch.arange(1, k).to(torch.int32)
    w = torch.rand(T, k, generator=g)
    per = E // world

    def local_forward(rows, local_ids, wts):
        assert local_ids.shape == (rows.shape[0], k) and int(local_ids.max()) < per and int(local_ids.min()) >= -1
        assert bool((local_ids >= 0).any(dim=1).all())                # no row was sent to a rank that owns none of its experts
        gids = torch.where(local_ids >= 0, local_ids + rank * per, torch.full_like(local_ids, -1))
        return _fake_layer(rows, gids, wts, rank * per, (rank + 1) * per)

    out = ep.ep_moe_forward(x, ids, w, E, local_forward)
    # the same arithmetic in one process: partial row per owner rank (rounded), added in rank order in FP32
    want = torch.zeros(T, K)
    for r in range(world):
        want += _fake_layer(x, ids, w, r * per, (r + 1) * per).float()
    ok = torch.equal(out, want.to(torch.bfloat16))

    # the all-gather / reduce-scatter formulation (every rank sees every token; rows without a local expert are
    # all -1 and must come back as zeros); the sum over ranks is the collective's, so allow one bf16 ulp
    def local_forward_all(rows, local_ids, wts):
        gids = torch.where(local_ids >= 0, local_ids + rank * per, torch.full_like(local_ids, -1))
        return _fake_layer(rows, gids, wts, rank * per, (rank + 1) * per)

    out2 = ep.ep_moe_forward_gathered(x, ids, w, E, local_forward_all)
    ok = ok and bool(((out2.float() - want).abs() <= 2.0 ** -7 * want.abs() + 1e-6).all())
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if int(flag) != 1:
        raise SystemExit(3)


@pytest.mark.parametrize("world,T", [(2, 17), (4, 5)])
def test_expert_parallel_bookkeeping(world, T):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, T, 8, 3, 16), nprocs=world, join=True)


def test_plan_dispatch_groups_by_owner():
    import __graft_entry__ as entry
    entry.load_package()
    ep = importlib.import_module("dsv4_b200.runtime.expert_parallel")
    ids = torch.tensor([[5, 0], [2, 3], [1, 6], [7, 4]], dtype=torch.int32)
    token_of, counts = ep.plan_dispatch(ids, 4, 2)
    assert counts.tolist() == [3, 3]                                   # token 1 only to rank 0, token 3 only to rank 1
    assert token_of.tolist() == [0, 1, 2, 0, 2, 3]                     # rank 0's rows, then rank 1's; tokens ascending
