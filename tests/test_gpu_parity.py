"""GPU parity: the CUDA libraries, called through their C ABI bindings, against the CPU oracle (and, when built,
against the reference's own CUDA kernels) on identical seeded inputs.

Acceptance rule (stated by the benchmark definition): dequantised weights bit-exact, expert selection identical,
GEMV / MoE outputs max|out-ref| <= 1e-2 * max|ref| and cosine >= 0.9999 against the FP32 reference.
"""
import numpy as np
import pytest
import torch

import oracle
from oracle import ref_kernels

pytestmark = pytest.mark.gpu

TOL_MAXABS = 1e-2
TOL_COS = 0.9999


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def accept(out_bf16, ref_f32, tight=True):
    out = out_bf16.float().cpu().numpy()
    err, cos = oracle.max_abs_rel(out, ref_f32), oracle.cosine(out, ref_f32)
    assert err <= TOL_MAXABS and cos >= TOL_COS, f"max-abs/inf {err:.3e} cosine {cos:.7f}"
    if tight:   # the kernels are far inside the rule: one bf16 rounding of an output is up to 2^-8 = 3.9e-3 of it
        assert err <= 5e-3 and cos >= 0.99999, f"(tight) max-abs/inf {err:.3e} cosine {cos:.7f}"
    return err, cos


def rand_mxfp4(qz, rows, cols, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)
    return qz.quantize_mxfp4(w)


def rand_x(k, seed):
    return torch.randn(k, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------------ dequantisation

def test_dequant_bit_exact_against_golden(rt, golden, dev):
    p = torch.from_numpy(golden["mxfp4_packed"]).to(dev)
    s = torch.from_numpy(golden["mxfp4_scale"]).to(dev)
    got = rt.mxfp4_dequant_bf16(p, s)
    bits = got.view(torch.int16).cpu().numpy()
    ref = golden["mxfp4_dequant_bf16_bits"]
    nan = np.isnan(got.float().cpu().numpy())
    ref_nan = np.isnan(torch.from_numpy(ref.copy()).view(torch.bfloat16).float().numpy())
    assert np.array_equal(nan, ref_nan) and nan.sum() == 32
    assert np.array_equal(bits[~nan], ref[~nan])      # bit patterns: -0.0 and subnormal scales included


def test_dequant_bit_exact_random(rt, dev):
    rng = np.random.default_rng(11)
    p = rng.integers(0, 256, size=(257, 512), dtype=np.uint8)
    s = rng.integers(0, 255, size=(257, 32), dtype=np.uint8)      # every non-NaN scale byte
    got = rt.mxfp4_dequant_bf16(torch.from_numpy(p).to(dev), torch.from_numpy(s).to(dev))
    want = oracle.bf16_bits(oracle.bf16_round(oracle.dequant_mxfp4(p, s)))
    assert np.array_equal(got.view(torch.int16).cpu().numpy(), want)


# ------------------------------------------------------------------------------------------------ MXFP4 dense GEMV

@pytest.mark.parametrize("K,N", [(32, 1), (64, 33), (128, 32), (1024, 7), (992, 65), (4096, 2048), (8192, 300)])
def test_mxfp4_gemv(rt, qz, dev, K, N):
    p, s = rand_mxfp4(qz, N, K, seed=K + N)
    x = rand_x(K, seed=K)
    y = rt.mxfp4_gemv(p.to(dev), s.to(dev), x.to(dev))
    # with a handful of outputs one bf16 rounding (2^-8 of the value) can be the whole max|ref|
    accept(y, oracle.mxfp4_gemv_ref(p, s, x), tight=N >= 32)
    if ref_kernels.available():
        y_ref = ref_kernels.mxfp4_gemv(x.to(dev), p.to(dev), s.to(dev))
        accept(y, y_ref.float().cpu().numpy(), tight=False)


def test_mxfp4_gemv_edge_scales_and_values(rt, dev):
    rng = np.random.default_rng(5)
    K, N = 256, 40
    p = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)        # every nibble incl. -0.0
    s = rng.integers(118, 130, size=(N, K // 32), dtype=np.uint8)
    s[0, :] = 255                  # NaN sentinel: contributes 0 in kernel semantics
    s[1, 0], s[1, 1] = 0, 250      # smallest (FP32-subnormal) scale and a huge one that still fits FP32
    s[2, :] = 0
    x = rand_x(K, 9)
    x[32:64] = 0                   # an all-zero activation block
    y = rt.mxfp4_gemv(torch.from_numpy(p).to(dev), torch.from_numpy(s).to(dev), x.to(dev))
    ref = oracle.mxfp4_gemv_ref(p, s, x)
    yc = y.float().cpu().numpy()
    assert yc[0] == 0.0
    assert np.isfinite(yc).all()
    np.testing.assert_allclose(yc[1], ref[1], rtol=1e-2)
    np.testing.assert_allclose(yc[3:], ref[3:], rtol=0, atol=4e-3 * np.abs(ref[3:]).max())


def test_mxfp4_gemv_strided_and_unaligned(rt, qz, dev):
    K, N = 512, 48
    p, s = rand_mxfp4(qz, 2 * N, K, seed=3)
    x = rand_x(K, 4)
    ref = oracle.mxfp4_gemv_ref(p[::2], s[::2], x)
    # every second row of a larger matrix: row stride 2x, still 16-byte aligned
    accept(rt.mxfp4_gemv(p.to(dev)[::2], s.to(dev)[::2], x.to(dev)), ref)
    # a view starting 1 byte into a buffer, rows 1 byte longer than the data: nothing is 16-byte aligned
    buf = torch.zeros(N * (K // 2 + 1) + 1, dtype=torch.uint8, device=dev)
    view = buf[1:].view(N, K // 2 + 1)[:, : K // 2]
    view.copy_(p[::2].to(dev))
    assert view.data_ptr() % 16 != 0 and view.stride(0) % 16 != 0
    accept(rt.mxfp4_gemv(view, s[::2].contiguous().to(dev), x.to(dev)), ref)


def test_mxfp4_gemv_rejects_bad_shapes(rt, dev):
    with pytest.raises(RuntimeError):
        rt.mxfp4_gemv(torch.zeros(4, 24, dtype=torch.uint8, device=dev), torch.zeros(4, 1, dtype=torch.uint8, device=dev),
                      torch.zeros(48, dtype=torch.bfloat16, device=dev))
    with pytest.raises(RuntimeError, match="returned -2"):
        rt.mxfp4_gemv(torch.zeros(4, 8192, dtype=torch.uint8, device=dev),
                      torch.zeros(4, 512, dtype=torch.uint8, device=dev),
                      torch.zeros(16384, dtype=torch.bfloat16, device=dev))
    empty = rt.mxfp4_gemv(torch.zeros(0, 32, dtype=torch.uint8, device=dev),
                          torch.zeros(0, 2, dtype=torch.uint8, device=dev),
                          torch.zeros(64, dtype=torch.bfloat16, device=dev))
    assert empty.shape == (0,)


# ------------------------------------------------------------------------------------------------ FP8 dense GEMV

def rand_fp8(qz, N, K, seed, kind="e8m0"):
    g = torch.Generator().manual_seed(seed)
    return qz.quantize_fp8_block128(torch.randn(N, K, generator=g) * 0.02, kind)


# shapes: the tile minimum, config 1 (4096 -> 8192), and the engine's call sites (1024 -> 32768, 8192 -> 4096)
@pytest.mark.parametrize("K,N", [(128, 128), (256, 512), (4096, 8192), (1024, 32768), (8192, 4096), (16384, 128)])
def test_fp8_gemv(rt, qz, dev, K, N):
    w, s = rand_fp8(qz, N, K, seed=K + N)
    x = rand_x(K, seed=N)
    y = rt.fp8_e4m3_gemv(w.to(dev), s.to(dev), x.to(dev))
    accept(y, oracle.fp8_gemv_ref(w, s, x))
    if ref_kernels.available() and N * K <= 4096 * 8192:
        y_ref = ref_kernels.fp8_gemv(x.to(dev), w.to(dev), s.to(dev))
        accept(y, y_ref.float().cpu().numpy(), tight=False)


def test_fp8_gemv_f32_scales(rt, qz, dev):
    K, N = 4096, 8192     # config 1 as worded: FP32 scale = amax / 448 per 128x128 block
    w, s = rand_fp8(qz, N, K, seed=1235, kind="f32")
    x = rand_x(K, 1235)
    y = rt.fp8_e4m3_gemv_f32scale(w.to(dev), s.to(dev), x.to(dev))
    deq = oracle.e4m3_to_f32(w.numpy()) * np.repeat(np.repeat(s.numpy(), 128, 0), 128, 1)
    accept(y, deq @ x.float().numpy())


def test_fp8_gemv_every_code_and_nan(rt, dev):
    rng = np.random.default_rng(2)
    K, N = 256, 128
    w = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
    w[w == 0x7F] = 0x7E
    w[w == 0xFF] = 0xFE
    w[0, :256] = np.arange(256, dtype=np.uint8)      # row 0 holds both NaN codes
    s = np.full((1, 2), 120, dtype=np.uint8)
    x = rand_x(K, 6)
    y = rt.fp8_e4m3_gemv(torch.from_numpy(w).to(dev), torch.from_numpy(s).to(dev), x.to(dev)).float().cpu().numpy()
    ref = oracle.fp8_gemv_ref(w, s, x)
    assert np.isnan(y[0]) and np.isnan(ref[0])
    np.testing.assert_allclose(y[1:], ref[1:], rtol=0, atol=4e-3 * np.abs(ref[1:]).max())


def test_fp8_gemv_strided_slice(rt, qz, dev):
    # the engine multiplies 128-row-aligned column slices of a wider matrix (8 groups of 4096 columns)
    K, N, groups = 512, 256, 3
    w, s = rand_fp8(qz, N, K * groups, seed=8)
    x = rand_x(K, 8)
    wd, sd = w.to(dev), s.to(dev)
    for g in range(groups):
        y = rt.fp8_e4m3_gemv(wd[:, g * K:(g + 1) * K], sd[:, g * K // 128:(g + 1) * K // 128], x.to(dev))
        accept(y, oracle.fp8_gemv_ref(w[:, g * K:(g + 1) * K], s[:, g * K // 128:(g + 1) * K // 128], x))


# ------------------------------------------------------------------------------------------------ routed experts

def stacked(bank, ids):
    idx = torch.as_tensor(ids, dtype=torch.long)
    return {k: v[idx].contiguous() for k, v in bank.items()}


def run_grouped(rt, bank_dev, x, r, dev):
    return rt.mxfp4_grouped_gemv({"packed": bank_dev["w1p"], "scale": bank_dev["w1s"]},
                                 {"packed": bank_dev["w3p"], "scale": bank_dev["w3s"]},
                                 {"packed": bank_dev["w2p"], "scale": bank_dev["w2s"]}, None, x.to(dev), r.to(dev))


# (1024, 1024), (2048, 1024), (4096, 2048): shapes served by the shared-memory ring kernels; the others by the
# register-streaming kernels
@pytest.mark.parametrize("K,H", [(32, 32), (64, 96), (256, 128), (512, 512), (1024, 992), (1024, 1024), (2048, 1024),
                                 (1024, 1536), (2048, 4096), (4096, 2048)])
def test_grouped_gemv(rt, qz, dev, K, H):
    bank = qz.make_expert_bank(6, K, H, "cpu", seed=K + H)
    x = rand_x(K, K)
    r = torch.softmax(torch.randn(6, generator=torch.Generator().manual_seed(H)), 0) * 1.5
    ref = oracle.grouped_gemv_ref(x, bank["w1p"], bank["w3p"], bank["w2p"], bank["w1s"], bank["w3s"], bank["w2s"], r)
    bd = {k: v.to(dev) for k, v in bank.items()}
    out = run_grouped(rt, bd, x, r, dev)
    accept(out, ref)
    # deterministic: fixed summation order, no float atomics
    assert torch.equal(out.view(torch.int16), run_grouped(rt, bd, x, r, dev).view(torch.int16))
    assert rt.device_status() == 0          # no bounded wait ran out
    if ref_kernels.available():
        y_ref = ref_kernels.grouped_gemv(x.to(dev), bd["w1p"], bd["w3p"], bd["w2p"], bd["w1s"], bd["w3s"], bd["w2s"],
                                         r.to(dev))
        accept(out, y_ref.float().cpu().numpy(), tight=False)


def test_grouped_gemv_ids_equals_stacked(rt, qz, dev):
    K, H, E = 512, 256, 16
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=77)
    bd = {k: v.to(dev) for k, v in bank.items()}
    x = rand_x(K, 1)
    ids = [11, 3, 15, 0, 7, 8]
    r = torch.rand(6, generator=torch.Generator().manual_seed(2))
    a = run_grouped(rt, {k: v.to(dev) for k, v in stacked(bank, ids).items()}, x, r, dev)
    b = rt.mxfp4_grouped_gemv_ids(bd, torch.tensor(ids, dtype=torch.int32, device=dev), x.to(dev), r.to(dev))
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # fewer experts than 6 through the index entry
    sub = rt.mxfp4_grouped_gemv_ids(bd, torch.tensor(ids[:2], dtype=torch.int32, device=dev), x.to(dev),
                                    r[:2].to(dev))
    st = stacked(bank, ids[:2])
    accept(sub, oracle.grouped_gemv_ref(x, st["w1p"], st["w3p"], st["w2p"], st["w1s"], st["w3s"], st["w2s"], r[:2]))


def test_grouped_gemv_error_codes(rt, qz, dev):
    bank = {k: v.to(dev) for k, v in qz.make_expert_bank(5, 64, 32, "cpu", seed=1).items()}
    with pytest.raises(RuntimeError, match="returned -4"):
        run_grouped(rt, bank, rand_x(64, 1), torch.ones(5), dev)


def test_grouped_gemv_linearity_in_router_weights(rt, qz, dev):
    # size-independent property at the full DSv4 shape: out(r) is linear in r
    K, H = 4096, 2048
    bank = {k: v.to(dev) for k, v in qz.make_expert_bank(6, K, H, dev, seed=4).items()}
    x = rand_x(K, 2)
    total = None
    for e in range(6):
        r = torch.zeros(6)
        r[e] = 0.25 + 0.1 * e
        y = run_grouped(rt, bank, x, r, dev).float()
        total = y if total is None else total + y
    r_all = torch.tensor([0.25 + 0.1 * e for e in range(6)])
    y_all = run_grouped(rt, bank, x, r_all, dev).float()
    err = (y_all - total).abs().max() / y_all.abs().max()
    assert err <= 1e-2      # each of the seven outputs carries its own bf16 rounding


# ------------------------------------------------------------------------------------------------ router

@pytest.mark.parametrize("func", ["sqrt_softplus", "softmax"])
def test_router_topk(rt, golden, dev, func):
    rng = np.random.default_rng(21)
    logits = np.concatenate([golden["route_logits"], rng.standard_normal((64, 256)).astype(np.float32)])
    ids, w = rt.moe_route_topk(torch.from_numpy(logits).to(dev), k=6, score_func=func)
    ids, w = ids.cpu().numpy(), w.cpu().numpy()
    if func == "sqrt_softplus":
        ref_ids, ref_w = oracle.route_sqrt_softplus(logits)
    else:
        ref_ids, ref_w = oracle.route_softmax(logits)
    distinct = np.array([len(np.unique(row)) == row.size for row in logits])
    assert np.array_equal(ids[distinct], ref_ids[distinct])            # identical expert selection
    np.testing.assert_allclose(w[distinct], ref_w[distinct], rtol=2e-6, atol=1e-30)
    # rows with tied logits: the same score multiset must be chosen, lowest indices first among equals
    for t in np.flatnonzero(~distinct):
        assert np.array_equal(np.sort(logits[t][ids[t]]), np.sort(logits[t][ref_ids[t]]))
    # against the reference's own _route output (golden): same experts on rows without ties
    g_ids = golden["route_ids"]
    for t in range(4):
        assert np.array_equal(ids[t], g_ids[t])


def test_router_other_shapes(rt, dev):
    rng = np.random.default_rng(8)
    for T, E, k in [(1, 256, 6), (3, 64, 2), (5, 8, 8), (2, 1000, 32)]:
        logits = rng.standard_normal((T, E)).astype(np.float32)
        ids, w = rt.moe_route_topk(torch.from_numpy(logits).to(dev), k=k, score_func="softmax")
        ref_ids, ref_w = oracle.route_softmax(logits, k)
        assert np.array_equal(ids.cpu().numpy(), ref_ids)
        np.testing.assert_allclose(w.cpu().numpy(), ref_w, rtol=2e-6)


# ------------------------------------------------------------------------------------------------ one-call layer

@pytest.mark.parametrize("K,H,E,func", [(1024, 1024, 32, "softmax"), (4096, 2048, 16, "sqrt_softplus"),
                                        (256, 128, 12, "softmax"), (1024, 1024, 300, "sqrt_softplus")])
def test_decode_layer_one_call(rt, qz, dev, K, H, E, func):
    """Router + FFN in one call (fused router at ring shapes, separate router kernel otherwise) against the oracle
    and, bit for bit, against the two-call sequence."""
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=E)
    bd = {k: v.to(dev) for k, v in bank.items()}
    x = rand_x(K, 3)
    logits = torch.randn(E, generator=torch.Generator().manual_seed(5))
    ws = torch.empty(rt.decode_workspace_bytes(6, H, K), dtype=torch.uint8, device=dev)
    out = rt.moe_decode_layer(bd, logits.to(dev), x.to(dev), k=6, score_func=func, workspace=ws)
    ids, w = rt.decode_picks(ws, 6, H)
    ref_ids, ref_w = (oracle.route_softmax if func == "softmax" else oracle.route_sqrt_softplus)(logits.numpy()[None])
    assert np.array_equal(ids.cpu().numpy(), ref_ids[0])                       # identical expert selection
    np.testing.assert_allclose(w.cpu().numpy(), ref_w[0], rtol=2e-6)
    st = stacked(bank, ref_ids[0].tolist())
    ref = oracle.grouped_gemv_ref(x, st["w1p"], st["w3p"], st["w2p"], st["w1s"], st["w3s"], st["w2s"], ref_w[0])
    accept(out, ref)
    ids2, w2 = rt.moe_route_topk(logits.to(dev), k=6, score_func=func)
    out2 = rt.mxfp4_grouped_gemv_ids(bd, ids2[0].contiguous(), x.to(dev), w2[0].contiguous())
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    assert rt.device_status() == 0
