"""GPU parity of the batched routed-expert layer (tcgen05 grouped GEMMs) against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def routing(T, E, k, seed, zipf=False):
    g = torch.Generator().manual_seed(seed)
    if zipf:
        p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** 1.1
        ids = torch.multinomial(p.expand(T, E), k, replacement=False, generator=g)
    else:
        ids = torch.rand(T, E, generator=g).topk(k).indices
    w = torch.softmax(torch.randn(T, k, generator=g), -1)
    return ids.to(torch.int32), w.float()


@pytest.mark.parametrize("path", ["mxf4", "fp16"])
@pytest.mark.parametrize("T,E,K,H,O,k,zipf", [
    (1, 4, 256, 256, 128, 2, False),          # a single token
    (20, 8, 256, 256, 256, 2, False),
    (64, 16, 512, 512, 384, 6, True),         # skewed: some experts get most tokens, some none
    (300, 3, 256, 512, 256, 2, False),        # more than 128 tokens per expert: several token tiles
])
def test_moe_forward_small(rt, qz, T, E, K, H, O, k, zipf, path):
    dev = torch.device("cuda:0")
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=T + E)
    if O != K:                                  # down projection to a different width
        g = torch.Generator().manual_seed(9)
        w2 = (torch.randn(E, O, H, generator=g) * 0.02).to(torch.bfloat16)
        bank["w2p"], bank["w2s"] = qz.quantize_mxfp4(w2)
    x = (torch.randn(T, K, generator=torch.Generator().manual_seed(1)) * 3.0).to(torch.bfloat16)
    ids, w = routing(T, E, k, seed=5, zipf=zipf)
    out = rt.moe_forward({n: v.to(dev) for n, v in bank.items()}, x.to(dev), ids.to(dev), w.to(dev), path=path)
    torch.cuda.synchronize()
    assert rt.moe_device_status() == 0
    ref = oracle.moe_layer_ref(x, bank, ids.numpy(), w.numpy())
    got = out.float().cpu().numpy()
    err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
    assert err <= 1e-2 and cos >= 0.9999, f"max-abs/inf {err:.3e} cosine {cos:.7f}"
    # the fp16 path has exact operands; the block-scaled path carries the 3-term MXFP4 error of the activations
    tight = (5e-3, 0.99999) if path == "fp16" else (7e-3, 0.99997)
    assert err <= tight[0] and cos >= tight[1], f"(tight) max-abs/inf {err:.3e} cosine {cos:.7f}"
    print(f"{path}: max-abs/inf {err:.3e} cosine {cos:.7f}")
    # deterministic
    again = rt.moe_forward({n: v.to(dev) for n, v in bank.items()}, x.to(dev), ids.to(dev), w.to(dev), path=path)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))


@pytest.mark.parametrize("path", ["mxf4", "fp16"])
def test_moe_forward_matches_single_token_path(rt, qz, path):
    """Batched decode at the DSv4 expert shape against the one-token decode kernel, token by token."""
    dev = torch.device("cuda:0")
    T, E, K, H, k = 8, 12, 4096, 2048, 6
    bank = {n: v for n, v in qz.make_expert_bank(E, K, H, dev, seed=3).items()}
    x = torch.randn(T, K, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(dev)
    ids, w = routing(T, E, k, seed=8)
    out = rt.moe_forward(bank, x, ids.to(dev), w.to(dev), path=path)
    for t in range(T):
        one = rt.mxfp4_grouped_gemv_ids(bank, ids[t].contiguous().to(dev), x[t].contiguous(), w[t].contiguous().to(dev))
        d = (out[t].float() - one.float()).abs().max() / one.float().abs().max()
        assert d <= 1e-2
    assert rt.moe_device_status() == 0


@pytest.mark.parametrize("path", ["mxf4", "fp16"])
def test_moe_forward_scale_invariance(rt, qz, path):
    """x scaled by 2^20 and 2^-20: the normalisation must keep fp16 operands in range; the output follows x
    through the SwiGLU (checked against the oracle on the scaled input)."""
    dev = torch.device("cuda:0")
    T, E, K, H, k = 16, 4, 256, 256, 2
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=2)
    ids, w = routing(T, E, k, seed=3)
    for scale in (2.0 ** 20, 2.0 ** -20):
        x = (torch.randn(T, K, generator=torch.Generator().manual_seed(4)) * scale).to(torch.bfloat16)
        out = rt.moe_forward({n: v.to(dev) for n, v in bank.items()}, x.to(dev), ids.to(dev), w.to(dev), path=path)
        ref = oracle.moe_layer_ref(x, bank, ids.numpy(), w.numpy())
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert oracle.max_abs_rel(got, ref) <= 1e-2 and oracle.cosine(got, ref) >= 0.9999


@pytest.mark.parametrize("path", ["mxf4", "fp16"])
def test_moe_forward_skips_negative_ids(rt, qz, path):
    """A negative id marks a pair to skip (how an expert-parallel rank masks the experts of other ranks): the result
    is the layer without those pairs (oracle with their router weight set to zero); a token whose pairs are all
    skipped gets zeros; the status word stays 0."""
    dev = torch.device("cuda:0")
    T, E, K, H, k = 40, 8, 256, 512, 4
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=21)
    x = (torch.randn(T, K, generator=torch.Generator().manual_seed(3)) * 2.0).to(torch.bfloat16)
    ids, w = routing(T, E, k, seed=6)
    g = torch.Generator().manual_seed(7)
    drop = torch.rand(T, k, generator=g) < 0.4
    drop[5] = True                                                   # token 5: nothing local
    masked = torch.where(drop, torch.full_like(ids, -1), ids)
    out = rt.moe_forward({n: v.to(dev) for n, v in bank.items()}, x.to(dev), masked.to(dev), w.to(dev), path=path)
    torch.cuda.synchronize()
    assert rt.moe_device_status() == 0
    w_kept = torch.where(drop, torch.zeros_like(w), w)
    ref = oracle.moe_layer_ref(x, bank, ids.numpy(), w_kept.numpy())
    got = out.float().cpu().numpy()
    err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
    assert err <= 1e-2 and cos >= 0.9999, f"max-abs/inf {err:.3e} cosine {cos:.7f}"
    assert not np.any(got[5])


def test_moe_forward_short_reduction_many_tiles(rt, qz):
    """hidden = 1024 (four 256-wide K steps per down tile) with several tiles per CTA: the token tables of three
    consecutive tiles are live at once in the block-scaled kernel."""
    dev = torch.device("cuda:0")
    T, E, K, H, O, k = 2048, 8, 512, 1024, 2048, 2
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=31)
    g = torch.Generator().manual_seed(32)
    w2 = (torch.randn(E, O, H, generator=g) * 0.02).to(torch.bfloat16)
    bank["w2p"], bank["w2s"] = qz.quantize_mxfp4(w2)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    ids, w = routing(T, E, k, seed=33)
    w = w * torch.linspace(0.25, 4.0, T)[:, None]            # router weights that differ a lot from tile to tile
    dbank = {n: v.to(dev) for n, v in bank.items()}
    ref = oracle.moe_layer_ref(x, bank, ids.numpy(), w.numpy())
    for path in ("mxf4", "fp16"):
        for rep in range(3):
            out = rt.moe_forward(dbank, x.to(dev), ids.to(dev), w.to(dev), path=path)
            torch.cuda.synchronize()
            got = out.float().cpu().numpy()
            err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
            assert err <= 1e-2 and cos >= 0.9999, f"{path} rep {rep}: max-abs/inf {err:.3e} cosine {cos:.7f}"
    assert rt.moe_device_status() == 0


@pytest.fixture(scope="module")
def full_bank(qz):
    dev = torch.device("cuda:0")
    bank = qz.make_expert_bank(256, 4096, 2048, dev, seed=1236, chunk=16)
    yield bank
    del bank
    torch.cuda.empty_cache()


@pytest.mark.parametrize("name,T,zipf,seed,n_sample", [("config3_decode_batch64_zipf", 64, True, 1237, 12),
                                                      ("config4_prefill_4096_uniform", 4096, False, 1238, 24)])
def test_configs_3_and_4_at_stated_size_against_the_oracle(rt, full_bank, name, T, zipf, seed, n_sample):
    """The batched configurations as stated (256 experts, K = 4096, hidden = 2048, top-6; 64 tokens with Zipf(1.1)
    routing, 4096 tokens with uniform routing) through the batched layer, a sample of tokens checked against the FP32
    CPU oracle (only the experts those tokens use are dequantised on the CPU)."""
    dev = torch.device("cuda:0")
    E, K, k = 256, 4096, 6
    g = torch.Generator().manual_seed(seed)
    if zipf:
        p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** 1.1
        ids = torch.multinomial(p.expand(T, E), k, replacement=False, generator=g)
    else:
        ids = torch.rand(T, E, generator=g).topk(k).indices
    w = torch.softmax(torch.randn(T, k, generator=g), -1).float()
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    out = rt.moe_forward(full_bank, x.to(dev), ids.to(torch.int32).to(dev), w.to(dev))
    torch.cuda.synchronize()
    assert rt.moe_device_status() == 0
    sample = torch.randperm(T, generator=g)[:n_sample].sort().values
    used = torch.unique(ids[sample])
    remap = {int(e): i for i, e in enumerate(used.tolist())}
    sub = {n: v[used.to(dev)].cpu() for n, v in full_bank.items()}
    ids_s = np.vectorize(remap.get)(ids[sample].numpy())
    ref = oracle.moe_layer_ref(x[sample], sub, ids_s, w[sample].numpy())
    got = out[sample.to(dev)].float().cpu().numpy()
    err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
    assert err <= 1e-2 and cos >= 0.9999, f"{name}: max-abs/inf {err:.3e} cosine {cos:.7f}"


def test_moe_forward_65536_tokens_small_dims(rt, qz):
    """More tokens than a grid dimension holds (the combine kernel walks tokens with a stride): 65 536 tokens at
    small dimensions, a sample of tokens against the oracle."""
    dev = torch.device("cuda:0")
    T, E, K, H, O, k = 65536, 4, 256, 256, 128, 1
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=41)
    g = torch.Generator().manual_seed(42)
    w2 = (torch.randn(E, O, H, generator=g) * 0.02).to(torch.bfloat16)
    bank["w2p"], bank["w2s"] = qz.quantize_mxfp4(w2)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    ids, w = routing(T, E, k, seed=43)
    out = rt.moe_forward({n: v.to(dev) for n, v in bank.items()}, x.to(dev), ids.to(dev), w.to(dev))
    torch.cuda.synchronize()
    assert rt.moe_device_status() == 0
    sample = torch.cat([torch.arange(0, 8), torch.arange(65528, 65536), torch.randint(0, T, (48,), generator=g)])
    ref = oracle.moe_layer_ref(x[sample], bank, ids[sample].numpy(), w[sample].numpy())
    got = out[sample.to(dev)].float().cpu().numpy()
    err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
    assert err <= 1e-2 and cos >= 0.9999, f"max-abs/inf {err:.3e} cosine {cos:.7f}"


def test_stage_timing_reports_six_stages_and_changes_nothing(rt, qz):
    dev = torch.device("cuda:0")
    T, E, K, H, k = 96, 8, 512, 512, 2
    bank = {n: v.to(dev) for n, v in qz.make_expert_bank(E, K, H, "cpu", seed=51).items()}
    x = torch.randn(T, K, generator=torch.Generator().manual_seed(52)).to(torch.bfloat16).to(dev)
    ids, w = routing(T, E, k, seed=53)
    plain = rt.moe_forward(bank, x, ids.to(dev), w.to(dev), path="mxf4")
    assert rt.stage_timing(True) is False
    try:
        timed = rt.moe_forward(bank, x, ids.to(dev), w.to(dev), path="mxf4")
        stages = rt.stage_times()
    finally:
        assert rt.stage_timing(False) is True
    assert list(stages) == list(rt.STAGES) and all(0.0 < v < 1e5 for v in stages.values()), stages
    assert torch.equal(plain.view(torch.int16), timed.view(torch.int16))


def test_mma_rate_probe(rt):
    """The library's tensor-pipe microbenchmark: a kind::mxf4 MMA of N = 256 takes longer than one of N = 64, scale
    copies add to it, and the numbers are of the order the hardware allows (tens to a few hundred clocks)."""
    n64, n256, n256_copies = rt.mma_clocks(64, 0, 500), rt.mma_clocks(256, 0, 500), rt.mma_clocks(256, 4, 500)
    assert 30.0 < n64 <= n256 * 1.05 and n256 < 400.0, (n64, n256)
    assert n256 < n256_copies < 1000.0, (n256, n256_copies)
    with pytest.raises(RuntimeError):
        rt.mma_clocks(250, 0, 10)                # N must be a multiple of 16
