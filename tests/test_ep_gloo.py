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
    return (rows.float() * (expert_global.float() + 1.0) * w).to(rows.dtype)


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
        return _fake_expert(rows, local_ids + rank * per, wts)

    out = ep.ep_moe_forward(x, ids, w, E, local_forward)
    want = torch.zeros(T, K)
    for j in range(k):
        want += _fake_expert(x, ids[:, j:j + 1], w[:, j:j + 1]).float()
    ok = torch.equal(out, want.to(torch.bfloat16))
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
    ids = torch.tensor([[5, 0], [2, 7], [1, 6]], dtype=torch.int32)
    order, counts, local = ep.plan_dispatch(ids, 4, 2)
    assert counts.tolist() == [3, 3]
    assert order.tolist() == [1, 2, 4, 0, 3, 5]                        # stable inside a destination
    assert local.tolist() == [0, 2, 1, 1, 3, 2]
