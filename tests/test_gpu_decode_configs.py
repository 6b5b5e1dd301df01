"""The routed decode layer at the benchmark's stated size, and the MXFP4 decode kernels under activations that
stress their arithmetic (fp16 products summed 16 at a time in fp16, FP32 beyond), against the FP32 CPU oracle.

Tolerance (the benchmark definition's): max|out - ref| <= 1e-2 * max|ref| and cosine >= 0.9999.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL_MAXABS = 1e-2
TOL_COS = 0.9999
K, H = 4096, 2048


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def check(out_bf16, ref_f32):
    out = out_bf16.float().cpu().numpy()
    assert np.isfinite(out).all()
    err, cos = oracle.max_abs_rel(out, ref_f32), oracle.cosine(out, ref_f32)
    assert err <= TOL_MAXABS and cos >= TOL_COS, f"max-abs/inf {err:.3e} cosine {cos:.7f}"
    return err, cos


def picked_on_cpu(bank_dev, ids):
    idx = torch.as_tensor(ids, dtype=torch.long, device=bank_dev["w1p"].device)
    return {k: v[idx].cpu() for k, v in bank_dev.items()}


def test_config2_as_stated_256_experts_softmax_top6(rt, qz, dev):
    """256-expert bank (3.42 GB, generated on the device), logits ~N(0,1), softmax, top-6 renormalised, through the
    one-call layer; the oracle dequantises the six picked experts on the CPU."""
    bank = qz.make_expert_bank(256, K, H, dev, seed=1236, chunk=16)
    g = torch.Generator().manual_seed(1236)
    ws = torch.empty(rt.decode_workspace_bytes(6, H, K), dtype=torch.uint8, device=dev)
    for step in range(3):
        x = torch.randn(K, generator=g).to(torch.bfloat16)
        logits = torch.randn(256, generator=g)
        out = rt.moe_decode_layer(bank, logits.to(dev), x.to(dev), k=6, score_func="softmax", workspace=ws)
        ids, w = rt.decode_picks(ws, 6, H)
        ref_ids, ref_w = oracle.route_softmax(logits.numpy()[None], 6)
        assert np.array_equal(ids.cpu().numpy(), ref_ids[0])                   # identical expert selection
        np.testing.assert_allclose(w.cpu().numpy(), ref_w[0], rtol=2e-6)
        st = picked_on_cpu(bank, ref_ids[0].tolist())
        ref = oracle.grouped_gemv_ref(x, st["w1p"], st["w3p"], st["w2p"], st["w1s"], st["w3s"], st["w2s"], ref_w[0])
        check(out, ref)
    assert rt.device_status() == 0
    del bank
    torch.cuda.empty_cache()


def adversarial_activations():
    g = torch.Generator().manual_seed(99)
    base = torch.randn(K, generator=g)
    cases = {}
    # a handful of entries 10^3 .. 10^4 times the rest, as in LLM hidden states
    x = base.clone()
    idx = torch.randperm(K, generator=g)[:8]
    x[idx] *= torch.logspace(3, 4, 8)
    cases["outliers_1e3_1e4"] = x
    # moderate outliers: large enough to dominate an fp16 chain, small enough not to dominate the sum
    x = base.clone()
    x[torch.randperm(K, generator=g)[:32]] *= 100.0
    cases["outliers_100x"] = x
    # magnitudes across the bf16 range
    cases["magnitudes_2^-20_2^20"] = base * torch.exp2(torch.randint(-20, 21, (K,), generator=g).float())
    # cancellation: a large alternating component that the weights mostly cancel, over a small signal
    sign = torch.ones(K)
    sign[1::2] = -1.0
    cases["cancellation"] = 50.0 * sign + base
    # everything tiny / everything huge (one scale for the whole vector must still work)
    cases["tiny_2^-30"] = base * 2.0 ** -30
    cases["huge_2^30"] = base * 2.0 ** 30
    return {k: v.to(torch.bfloat16) for k, v in cases.items()}


@pytest.fixture(scope="module")
def small_bank(qz):
    return qz.make_expert_bank(8, K, H, "cpu", seed=4242)


@pytest.mark.parametrize("name", list(adversarial_activations().keys()))
@pytest.mark.parametrize("mode", ["pdl", "chain"])
def test_adversarial_activations_dsv4_shape(rt, dev, small_bank, name, mode):
    """Both decode paths (the single kernel and the two-kernel chain) at (4096, 2048)."""
    import importlib
    gb = importlib.import_module("dsv4_b200.runtime.mxfp4_grouped_gemv_binding")
    x = adversarial_activations()[name]
    bank = small_bank
    bd = {k: v.to(dev) for k, v in bank.items()}
    ids = [5, 0, 7, 2, 3, 6]
    r = torch.softmax(torch.randn(6, generator=torch.Generator().manual_seed(1)), 0)
    st = {k: v[torch.as_tensor(ids)] for k, v in bank.items()}
    ref = oracle.grouped_gemv_ref(x, st["w1p"], st["w3p"], st["w2p"], st["w1s"], st["w3s"], st["w2s"], r)
    before = gb.set_launch_mode(mode)
    try:
        out = rt.mxfp4_grouped_gemv_ids(bd, torch.tensor(ids, dtype=torch.int32, device=dev), x.to(dev), r.to(dev))
        torch.cuda.synchronize()
    finally:
        gb.set_launch_mode(before)
    check(out, ref)
    assert rt.device_status() == 0


def test_output_stored_straight_into_pinned_host_memory(rt, dev, small_bank):
    """`out` may be pinned host memory (mapped on the device): the kernel's own stores are the device-to-host
    transfer.  Bitwise equal to the output written to device memory."""
    bank = {k: v.to(dev) for k, v in small_bank.items()}
    g = torch.Generator().manual_seed(77)
    x = torch.randn(K, generator=g).to(torch.bfloat16).to(dev)
    logits = torch.randn(8, generator=g).to(dev)
    ws = torch.empty(rt.decode_workspace_bytes(6, H, K), dtype=torch.uint8, device=dev)
    on_device = rt.moe_decode_layer(bank, logits, x, k=6, score_func="softmax", workspace=ws).clone()
    host = torch.full((K,), float("nan"), dtype=torch.bfloat16).pin_memory()
    rt.moe_decode_layer(bank, logits, x, k=6, score_func="softmax", out=host, workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(host.view(torch.int16), on_device.cpu().view(torch.int16))
    assert rt.device_status() == 0
