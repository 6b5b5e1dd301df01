"""Two contracts of the single-kernel decode path (csrc/decode_stream.cuh) that parity tests do not reach:

* re-entrancy: what its CTAs wait on lives in the caller's workspace, so two calls on two streams with two
  workspaces may overlap on the device and still give the bits of the same calls run one after the other;
* the give-up path of its bounded waits: a wait that cannot be satisfied ends after its poll budget, the kernel
  returns, the status is reported, the output rows are NaN, and the next ordinary call is bit-exact again.
  The unsatisfiable wait is made on the host side of the call (the service warps are told to expect tags that no
  producer writes); nothing faults, traps or spins without a limit.
"""
import importlib

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

K, H, E, k = 4096, 2048, 24, 6


@pytest.fixture(scope="module")
def case(qz):
    dev = torch.device("cuda:0")
    bank = qz.make_expert_bank(E, K, H, dev, seed=321)
    g = torch.Generator(device=dev).manual_seed(7)
    xs = [torch.randn(K, generator=g, device=dev).to(torch.bfloat16) for _ in range(8)]
    logits = [torch.randn(E, generator=g, device=dev) for _ in range(8)]
    return dev, bank, xs, logits


def test_two_streams_two_workspaces_equal_serial_calls(rt, case):
    """Default launch mode.  The two streams are released together by an event, so their grids are in flight at
    the same time; each call has its own workspace, which is all the entry's contract asks for."""
    dev, bank, xs, logits = case
    gb = importlib.import_module("dsv4_b200.runtime.mxfp4_grouped_gemv_binding")
    n = len(xs)
    serial = [rt.moe_decode_layer(bank, logits[i], xs[i], k=k, score_func="softmax").clone() for i in range(n)]
    torch.cuda.synchronize()
    ws = [torch.empty(rt.decode_workspace_bytes(k, H, K), dtype=torch.uint8, device=dev) for _ in range(2)]
    outs = [torch.empty(K, dtype=torch.bfloat16, device=dev) for _ in range(n)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
    for rep in range(3):
        go = torch.cuda.Event()
        blocker = torch.empty(1 << 26, dtype=torch.float32, device=dev)
        blocker.normal_()                       # some work on the default stream in front of the event
        go.record()
        for s, stream in enumerate(streams):
            with torch.cuda.stream(stream):
                stream.wait_event(go)
                for i in range(s, n, 2):        # stream 0: even calls, stream 1: odd calls, each with its own workspace
                    rt.moe_decode_layer(bank, logits[i], xs[i], k=k, score_func="softmax", out=outs[i], workspace=ws[s])
        torch.cuda.synchronize()
        for i in range(n):
            assert torch.equal(outs[i].view(torch.int16), serial[i].view(torch.int16)), (rep, i)
    assert gb.device_status() == 0


def test_bounded_wait_gives_up_reports_and_recovers(rt, case):
    dev, bank, xs, logits = case
    gb = importlib.import_module("dsv4_b200.runtime.mxfp4_grouped_gemv_binding")
    ws = torch.empty(rt.decode_workspace_bytes(k, H, K), dtype=torch.uint8, device=dev)
    good = rt.moe_decode_layer(bank, logits[0], xs[0], k=k, score_func="softmax", workspace=ws).clone()
    torch.cuda.synchronize()
    assert gb.device_status() == 0
    gb.debug_wait_limits(2000, 1)               # 2000 polls, and tags that no producer writes
    try:
        bad = rt.moe_decode_layer(bank, logits[0], xs[0], k=k, score_func="softmax", workspace=ws).clone()
        torch.cuda.synchronize()                # the kernel has returned: its waits ran out, it did not hang
    finally:
        gb.debug_wait_limits(0, 0)
    assert gb.device_status() == 3              # reported ...
    assert gb.device_status() == 0              # ... and cleared by the read
    assert torch.isnan(bad.float()).all()       # the damage is visible in the output, not silent
    again = rt.moe_decode_layer(bank, logits[0], xs[0], k=k, score_func="softmax", workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(again.view(torch.int16), good.view(torch.int16))
    ids, w = oracle.route_softmax(logits[0].cpu().numpy()[None], k)
    sub = {n_: v[torch.from_numpy(ids[0].astype(np.int64)).to(dev)].cpu() for n_, v in bank.items()}
    ref = oracle.moe_layer_ref(xs[0].cpu()[None], sub, np.arange(k)[None], w)[0]
    got = again.float().cpu().numpy()
    assert oracle.max_abs_rel(got, ref) <= 1e-2 and oracle.cosine(got, ref) >= 0.9999
    assert gb.device_status() == 0
