"""Expert parallel on real GPUs (NCCL, two ranks, one process per GPU): the three formulations (all-to-all, all-gather +
reduce-scatter, all-gather + combine fused with peer stores) against the single-GPU layer on the same tokens.  Skipped on a box with fewer than two GPUs."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import importlib, os, sys
import torch, torch.distributed as dist
sys.path.insert(0, {root!r})
import __graft_entry__ as entry
entry.load_package()
rt = importlib.import_module("dsv4_b200.runtime")
qz = importlib.import_module("dsv4_b200.runtime.quantize")
ep = importlib.import_module("dsv4_b200.runtime.expert_parallel")
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
E, K, H, k, T = 16, 512, 256, 4, 48                      # T tokens per rank
bank = qz.make_expert_bank(E, K, H, dev, seed=5)          # same bank on every rank
local_bank = ep.shard_bank(bank, rank, world)
g = torch.Generator().manual_seed(100 + rank)
x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(dev)
ids = torch.rand(T, E, generator=g).topk(k).indices.to(torch.int32).to(dev)
w = torch.softmax(torch.randn(T, k, generator=g), -1).float().to(dev)
ref = rt.moe_forward(bank, x, ids, w).float()
fwd = lambda rows, lids, wts: rt.moe_forward(local_bank, rows, lids, wts)
for name, fn in (("all_to_all", ep.ep_moe_forward), ("gathered", ep.ep_moe_forward_gathered)):
    out = fn(x, ids, w, E, fwd).float()
    err = float((out - ref).abs().max() / ref.abs().max())
    assert err <= 1e-2, (name, err)
ctx = ep.PeerCombine(T, K, dev)
for rep in range(3):                                      # alternating receive buffers, one barrier per call
    out = ep.ep_moe_forward_peer(ctx, x, ids, w, E, local_bank).float()
    err = float((out - ref).abs().max() / ref.abs().max())
    assert err <= 1e-2, ("peer", rep, err)
    again = ep.ep_moe_forward_peer(ctx, x, ids, w, E, local_bank)
    assert torch.equal(again.view(torch.int16), out.to(torch.bfloat16).view(torch.int16))
ctx2 = ep.PeerCombine(T, K, dev, in_dim=K, k=k)
for rep in range(3):                                      # inputs read from the peers' published buffers too
    out = ep.ep_moe_forward_peer_inputs(ctx2, x, ids, w, E, local_bank).float()
    err = float((out - ref).abs().max() / ref.abs().max())
    assert err <= 1e-2, ("peer inputs", rep, err)
torch.cuda.synchronize()
assert rt.moe_device_status() == 0
dist.barrier()
dist.destroy_process_group()
print("ok")
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_gpus():
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD.format(root=ROOT)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    for p, o in zip(procs, outs):
        assert p.returncode == 0 and o.strip().splitlines()[-1] == "ok", o[-3000:]
