"""GPU parity of fp8_e4m3_gemv_batched (several tokens / several independent groups in one launch) against the CPU
oracle and against the loop of single-token fp8_e4m3_gemv calls it replaces (bit for bit with one token, where the
same kernel runs per group; to rounding with several tokens, where the sums are formed by FP32 tensor-core MMAs):
the per-token loop of the reference's `_fp8_linear` (runtime/dsv4_engine_mxfp4.py:310-320) and the per-group loop of
the grouped output projection (kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:484-498).  Shapes are the attention projections'
(K -> N): wq_a 4096 -> 1024, wq_b 1024 -> 32768, wkv 4096 -> 512, wo_a 8 x (4096 -> 1024), wo_b 8192 -> 4096."""
from ctypes import c_int, c_int64

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def make(qz, rows, K, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return qz.quantize_fp8_block128(torch.randn(rows, K, generator=g) * std, "e8m0")


def bits(t):
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("name,K,N,G,S", [
    ("wq_a", 4096, 1024, 1, 1),
    ("wq_a", 4096, 1024, 1, 3),
    ("wkv", 4096, 512, 1, 2),
    ("wkv", 4096, 512, 1, 7),
    ("wq_b", 1024, 32768, 1, 4),
    ("wo_a", 4096, 1024, 8, 1),
    ("wo_a", 4096, 1024, 8, 2),
    ("wo_a", 4096, 1024, 8, 5),
    ("wo_b", 8192, 4096, 1, 9),
    ("wo_b", 8192, 4096, 1, 17),
    ("long_k", 16384, 256, 1, 3),
    ("odd_k", 2048 + 384, 128, 2, 8),
    ("small", 128, 128, 3, 6),
    ("ragged", 384, 640, 2, 2),
])
def test_batched_matches_oracle_and_single_calls(rt, qz, name, K, N, G, S):
    w, s = make(qz, G * N, K, seed=K + N + G)
    x = torch.randn(S, G * K, generator=torch.Generator().manual_seed(S)).to(torch.bfloat16)
    wd, sd, xd = w.to(DEV), s.to(DEV), x.to(DEV)
    y = rt.fp8_e4m3_gemv_batched(wd, sd, xd, n_groups=G)
    torch.cuda.synchronize()
    assert tuple(y.shape) == (S, G * N) and y.dtype == torch.bfloat16
    for t in range(S):
        for g in range(G):
            one = rt.fp8_e4m3_gemv(wd[g * N:(g + 1) * N], sd[g * N // 128:(g + 1) * N // 128],
                                   xd[t, g * K:(g + 1) * K].contiguous())
            got = y[t, g * N:(g + 1) * N]
            if S == 1:
                assert torch.equal(bits(one), bits(got)), f"{name}: group {g} differs from the single call"
            else:
                # both are bf16 roundings of sums that differ in the last FP32 bits: at most one bf16 step apart
                d = (one.float() - got.float()).abs().max() / one.float().abs().max()
                assert float(d) <= 2.0 ** -7, f"{name}: token {t} group {g}: {float(d):.3e} from the single call"
    # the oracle on a bounded number of (token, group) pairs: the comparison above carries the rest
    for t, g in {(0, 0), (S - 1, G - 1), (S // 2, G // 2)}:
        ref = oracle.fp8_gemv_ref(w[g * N:(g + 1) * N], s[g * N // 128:(g + 1) * N // 128], x[t, g * K:(g + 1) * K])
        got = y[t, g * N:(g + 1) * N].float().cpu().numpy()
        err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
        assert err <= 1e-2 and cos >= 0.9999, f"{name}: max-abs/inf {err:.3e} cosine {cos:.7f}"


def test_one_dimensional_input_and_out_argument(rt, qz):
    K, N, G = 4096, 1024, 8
    w, s = make(qz, G * N, K, seed=3)
    wd, sd = w.to(DEV), s.to(DEV)
    x = torch.randn(G * K, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    y = rt.fp8_e4m3_gemv_batched(wd, sd, x, n_groups=G)
    assert tuple(y.shape) == (G * N,)
    out = torch.zeros(G * N, dtype=torch.bfloat16, device=DEV)
    again = rt.fp8_e4m3_gemv_batched(wd, sd, x, n_groups=G, out=out)
    assert again.data_ptr() == out.data_ptr() and torch.equal(bits(out), bits(y))


def test_token_strides_wider_than_a_row(rt, qz):
    """x and y may be column slices of wider buffers (unit inner stride, 16-byte aligned token stride)."""
    K, N, S = 512, 256, 5
    w, s = make(qz, N, K, seed=5)
    wd, sd = w.to(DEV), s.to(DEV)
    xw = torch.randn(S, K + 64, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    yw = torch.full((S, N + 128), 7.0, dtype=torch.bfloat16, device=DEV)
    rt.fp8_e4m3_gemv_batched(wd, sd, xw[:, :K], out=yw[:, :N])
    want = rt.fp8_e4m3_gemv_batched(wd, sd, xw[:, :K].contiguous())
    assert torch.equal(bits(yw[:, :N]), bits(want))
    assert bool((yw[:, N:] == 7.0).all()), "columns beyond N must stay untouched"


def test_activation_magnitudes_across_the_bf16_range(rt, qz):
    """Tokens of very different magnitude in one pass: every (token, 2048-element half) carries its own power-of-two
    scale into the fp16 operands, so each row must match the single-token operator as closely as at unit scale."""
    K, N = 4096, 512
    w, s = make(qz, N, K, seed=11)
    wd, sd = w.to(DEV), s.to(DEV)
    scales = [1e-30, 1e-6, 1.0, 3e4, 1e20, 1e30, 0.0]
    x = torch.randn(len(scales), K, generator=torch.Generator().manual_seed(12))
    # one outlier per row: the rest of the row sits 2^10 below the largest magnitude
    x[:, 7] *= 1024.0
    x = (x * torch.tensor(scales).unsqueeze(1)).to(torch.bfloat16).to(DEV)
    y = rt.fp8_e4m3_gemv_batched(wd, sd, x)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(y.float()).all())
    for t, sc in enumerate(scales):
        one = rt.fp8_e4m3_gemv(wd, sd, x[t].contiguous()).float()
        if sc == 0.0:
            assert bool((y[t] == 0).all())
            continue
        d = (one - y[t].float()).abs().max() / one.abs().max()
        assert float(d) <= 2.0 ** -7, f"scale {sc:g}: {float(d):.3e} from the single call"


def test_return_codes(rt, qz):
    from importlib import import_module
    capi = import_module(rt.__name__ + "._capi")
    lib = capi.load("fp8")
    K, N = 256, 128
    w, s = make(qz, N, K, seed=8)
    wd, sd = w.to(DEV), s.to(DEV)
    x = torch.zeros(2, K, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(2, N, dtype=torch.bfloat16, device=DEV)

    def call(K_=K, N_=N, G=1, S=2, xs=K, ys=N, xp=None, ws=K):
        return lib.fp8_e4m3_gemv_batched(capi.ptr(x) if xp is None else xp, capi.ptr(wd), capi.ptr(sd), c_int(K_),
                                         c_int(N_), c_int64(ws), c_int64(K // 128), c_int(G), c_int(S), c_int64(xs),
                                         c_int64(ys), capi.ptr(y), capi.stream_ptr(DEV, None))

    assert call() == 0
    assert call(K_=100) == -1
    assert call(N_=100) == -2
    assert call(K_=16384 + 128) == -3
    assert call(G=0) == -8
    assert call(S=-1) == -8
    assert call(xs=K - 8) == -8          # token stride shorter than a row
    assert call(xs=K + 4) == -8          # token stride not 16-byte aligned
    assert call(xp=x.data_ptr() + 2) == -8
    assert call(S=0) == 0 and call(N_=0, ys=0) == 0
    with pytest.raises(RuntimeError):
        rt.fp8_e4m3_gemv_batched(wd, sd, x, n_groups=3)
    torch.cuda.synchronize()
