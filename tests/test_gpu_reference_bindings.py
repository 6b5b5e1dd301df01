"""The reference's OWN, unmodified ctypes bindings (runtime/mxfp4_grouped_gemv_binding.py, mxfp4_gemv_binding.py,
fp8_e4m3_gemv_binding.py of the reference tree) loaded against this repository's libraries through the environment
variables they read (MXFP4_GROUPED_LIB :31-36, MXFP4_GEMV_LIB :18-23, FP8_E4M3_GEMV_LIB :28-33), results checked
against the CPU oracle.  The reference tree is found through DSV4_REFERENCE_ROOT (default /root/reference); the test
is skipped where that tree does not exist (it never travels with the repository)."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REF_ROOT = os.environ.get("DSV4_REFERENCE_ROOT", "/root/reference")
HAVE_REF = os.path.isdir(os.path.join(REF_ROOT, "runtime"))


@pytest.mark.skipif(not HAVE_REF, reason="reference tree not present (set DSV4_REFERENCE_ROOT)")
def test_reference_bindings_load_the_new_libraries(pkg, qz):
    dev = torch.device("cuda:0")
    os.environ["MXFP4_GROUPED_LIB"] = pkg.lib_path("grouped")
    os.environ["MXFP4_GEMV_LIB"] = pkg.lib_path("mxfp4")
    os.environ["FP8_E4M3_GEMV_LIB"] = pkg.lib_path("fp8")
    sys.path.insert(0, REF_ROOT)
    try:
        grouped = importlib.import_module("runtime.mxfp4_grouped_gemv_binding")
        dense = importlib.import_module("runtime.mxfp4_gemv_binding")
        fp8 = importlib.import_module("runtime.fp8_e4m3_gemv_binding")
    finally:
        sys.path.remove(REF_ROOT)
    # routed experts: six stacked experts at the DSv4 shape
    K, H = 4096, 2048
    bank = qz.make_expert_bank(6, K, H, "cpu", seed=12)
    x = torch.randn(K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    r = torch.softmax(torch.randn(6, generator=torch.Generator().manual_seed(4)), 0)
    d = {n: v.to(dev) for n, v in bank.items()}
    out = grouped.mxfp4_grouped_gemv({"packed": d["w1p"], "scale": d["w1s"]}, {"packed": d["w3p"], "scale": d["w3s"]},
                                     {"packed": d["w2p"], "scale": d["w2s"]}, None, x.to(dev), r.to(dev))
    torch.cuda.synchronize()
    ref = oracle.grouped_gemv_ref(x, bank["w1p"], bank["w3p"], bank["w2p"], bank["w1s"], bank["w3s"], bank["w2s"], r)
    got = out.float().cpu().numpy()
    assert oracle.max_abs_rel(got, ref) <= 1e-2 and oracle.cosine(got, ref) >= 0.9999
    # dense MXFP4 and FP8 GEMVs
    wp, ws = qz.quantize_mxfp4((torch.randn(2048, K, generator=torch.Generator().manual_seed(5)) * 0.02).to(torch.bfloat16))
    y = dense.mxfp4_gemv(wp.to(dev), ws.to(dev), x.to(dev))
    assert oracle.max_abs_rel(y.float().cpu().numpy(), oracle.mxfp4_gemv_ref(wp, ws, x)) <= 1e-2
    wq, sq = qz.quantize_fp8_block128(torch.randn(1024, K, generator=torch.Generator().manual_seed(6)) * 0.02, "e8m0")
    y8 = fp8.fp8_e4m3_gemv(wq.to(dev), sq.to(dev), x.to(dev))
    assert oracle.max_abs_rel(y8.float().cpu().numpy(), oracle.fp8_gemv_ref(wq, sq, x)) <= 1e-2
