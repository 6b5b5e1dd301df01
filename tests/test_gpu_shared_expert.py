"""GPU parity of the fused FP8 shared-expert FFN (fp8_e4m3_shared_swiglu_m1) against the CPU oracle, under the two
clamp rules of the reference (C++ engine: gate only; Python engine: gate and up), and against the composition of
three fp8_e4m3_gemv calls it replaces."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def make_shared(qz, K, H, O, seed, std):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, rows, cols in (("w1", H, K), ("w3", H, K), ("w2", O, H)):
        w, s = qz.quantize_fp8_block128(torch.randn(rows, cols, generator=g) * std, "e8m0")
        out[name], out[name + "s"] = w, s
    return out


@pytest.mark.parametrize("K,H,O,std,xs", [
    (4096, 2048, 4096, 0.02, 1.0),         # the DSv4 shared expert
    (512, 256, 384, 0.05, 1.0),
    (4096, 2048, 4096, 0.06, 4.0),         # large pre-activations: the clamp at 10 bites
])
@pytest.mark.parametrize("limits", [(10.0, 0.0), (10.0, 10.0), (0.0, 0.0)])
def test_shared_swiglu_parity(rt, qz, K, H, O, std, xs, limits):
    dev = torch.device("cuda:0")
    shared = make_shared(qz, K, H, O, seed=K + H, std=std)
    x = (torch.randn(K, generator=torch.Generator().manual_seed(4)) * xs).to(torch.bfloat16)
    d = {n: v.to(dev) for n, v in shared.items()}
    out = rt.fp8_shared_swiglu(d, x.to(dev), limit_gate=limits[0], limit_up=limits[1])
    torch.cuda.synchronize()
    ref = oracle.shared_swiglu_fp8_ref(x, shared, limits[0], limits[1])
    got = out.float().cpu().numpy()
    err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
    # g, u and the activation are rounded to bf16 between the stages, as in the reference: three roundings of 2^-9
    assert err <= 1e-2 and cos >= 0.9999, f"max-abs/inf {err:.3e} cosine {cos:.7f}"
    if limits == (10.0, 0.0) and xs > 1.0:
        g = oracle.fp8_gemv_ref(shared["w1"], shared["w1s"], x)
        assert np.abs(g).max() > 10.0, "this case is meant to exercise the clamp"
    # deterministic
    again = rt.fp8_shared_swiglu(d, x.to(dev), limit_gate=limits[0], limit_up=limits[1])
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))


def test_shared_swiglu_equals_three_gemvs(rt, qz):
    """Bit for bit the composition the reference runs: bf16 GEMV outputs, clamp of the gate, bf16 activation, GEMV."""
    dev = torch.device("cuda:0")
    K, H, O = 4096, 2048, 4096
    shared = {n: v.to(dev) for n, v in make_shared(qz, K, H, O, seed=9, std=0.03).items()}
    x = (torch.randn(K, generator=torch.Generator().manual_seed(6)) * 2.0).to(torch.bfloat16).to(dev)
    fused = rt.fp8_shared_swiglu(shared, x, limit_gate=10.0, limit_up=0.0)
    g = rt.fp8_e4m3_gemv(shared["w1"], shared["w1s"], x).float().clamp(-10.0, 10.0)
    u = rt.fp8_e4m3_gemv(shared["w3"], shared["w3s"], x).float()
    act = (g / (1.0 + torch.exp(-g)) * u).to(torch.bfloat16)
    want = rt.fp8_e4m3_gemv(shared["w2"], shared["w2s"], act)
    d = (fused.float() - want.float()).abs().max() / want.float().abs().max()
    assert float(d) <= 4e-3, float(d)      # the activation may differ by one bf16 ulp (expf on the device vs torch.exp)


def test_shared_swiglu_errors(rt, qz):
    dev = torch.device("cuda:0")
    shared = {n: v.to(dev) for n, v in make_shared(qz, 256, 128, 256, seed=1, std=0.05).items()}
    x = torch.zeros(256, dtype=torch.bfloat16, device=dev)
    bad = dict(shared, w2s=shared["w2s"][:1])
    with pytest.raises(RuntimeError):
        rt.fp8_shared_swiglu(bad, x)
    with pytest.raises(RuntimeError):
        rt.fp8_shared_swiglu(shared, x, workspace=torch.empty(16, dtype=torch.uint8, device=dev))
    out = rt.fp8_shared_swiglu(shared, x)
    assert not bool(out.float().abs().max())               # zero input, zero output
