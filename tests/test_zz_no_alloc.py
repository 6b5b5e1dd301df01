"""The workspace-free entry point `mxfp4_grouped_gemv_topk_static`, called through the C ABI.

It exists for hosts that cannot obtain device memory when they call (all HBM already committed to the expert bank
and the KV cache, or a thread that must not enter cudaMalloc): the SwiGLU intermediate sits in a fixed array inside
the library instead of a caller-provided workspace.  The check: its output equals the workspace entry's, bit for
bit (same kernels, same summation order; the acceptance tolerance of the other GPU tests is asserted as well), on
two consecutive calls with different inputs - the array keeps the first call's contents, and the second call must
not be disturbed by them.  This file sorts last so that a run stopping at the first failure has already run every
other test; it does not depend on them.
"""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _case(qz, dev, K, H, seed):
    bank = qz.make_expert_bank(6, K, H, "cpu", seed=seed)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(K, generator=g).to(torch.bfloat16)
    r = torch.softmax(torch.randn(6, generator=g), 0) * 1.5
    return bank, x, r


def _sets(bank_dev):
    return ({"packed": bank_dev["w1p"], "scale": bank_dev["w1s"]}, {"packed": bank_dev["w3p"], "scale": bank_dev["w3s"]},
            {"packed": bank_dev["w2p"], "scale": bank_dev["w2s"]})


@pytest.mark.parametrize("K,H", [(4096, 2048), (256, 96)])      # the ring kernels and the register-streaming ones
def test_static_entry_matches_workspace_entry_twice(rt, qz, K, H):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dev = torch.device("cuda:0")
    out = torch.empty(K, dtype=torch.bfloat16, device=dev)
    for seed in (101, 202):                                       # two calls in a row on the shared array
        bank, x, r = _case(qz, dev, K, H, seed)
        bd = {k: v.to(dev) for k, v in bank.items()}
        w1, w3, w2 = _sets(bd)
        want = rt.mxfp4_grouped_gemv(w1, w3, w2, None, x.to(dev), r.to(dev))
        got = rt.mxfp4_grouped_gemv_static(w1, w3, w2, x.to(dev), r.to(dev), out)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        ref = oracle.grouped_gemv_ref(x, bank["w1p"], bank["w3p"], bank["w2p"], bank["w1s"], bank["w3s"], bank["w2s"], r)
        assert oracle.max_abs_rel(got.float().cpu(), ref) <= 1e-2 and oracle.cosine(got.float().cpu(), ref) >= 0.9999
    assert rt.device_status() == 0


def test_static_entry_rejects_sizes_beyond_its_scratch(rt):
    import ctypes
    import importlib
    lib = importlib.import_module("dsv4_b200.runtime._capi").load("grouped")
    one = ctypes.c_void_p(16)                                      # never dereferenced: the size check comes first
    assert lib.mxfp4_grouped_gemv_topk_static(*([one] * 8), 4096, 8192, 4096, 6, one, None) == -10
    assert lib.mxfp4_grouped_gemv_topk_static(*([one] * 8), 4096, 2048, 4096, 7, one, None) == -10
