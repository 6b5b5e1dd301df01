"""The synthetic-weight quantisers against the oracle's dequantisation (CPU)."""
import numpy as np
import torch

import oracle


def test_mxfp4_quantiser_rule(qz):
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(16, 256, generator=g) * 0.02).to(torch.bfloat16)
    packed, scale = qz.quantize_mxfp4(w)
    assert packed.shape == (16, 128) and scale.shape == (16, 8)
    blocks = w.float().reshape(16, 8, 32)
    amax = blocks.abs().amax(-1)
    expect = (torch.floor(torch.log2(amax)) - 2 + 127).to(torch.uint8)
    assert torch.equal(scale, expect)
    deq = oracle.dequant_mxfp4(packed, scale)
    # within a block the grid step is at most 2 * 2^e (between 4 and 6); values above 6 * 2^e saturate
    step = (2.0 ** (scale.float() - 127))[..., None]
    err = np.abs(deq.reshape(16, 8, 32) - blocks.numpy())
    sat = blocks.abs().numpy() > 6 * step.numpy()
    assert (err[~sat] <= step.numpy().repeat(32, -1)[~sat] + 1e-12).all()
    assert (np.abs(deq) <= 6 * step.numpy().repeat(32, -1).reshape(16, 256)).all()


def test_mxfp4_quantiser_is_exact_on_representable_values(qz):
    vals = torch.tensor(oracle.FP4_E2M1_VALUES).repeat(2)          # 32 values incl. -0.0, amax 6 -> e = 0
    packed, scale = qz.quantize_mxfp4(vals.reshape(1, 32))
    assert int(scale[0, 0]) == 127
    back = oracle.unpack_fp4(packed.numpy(), (32,))
    assert np.array_equal(back.view(np.uint32), vals.numpy().view(np.uint32))
    # ties go to the even code: 0.25 -> 0, 0.75 -> 1, 1.25 -> 1, 1.75 -> 2, 2.5 -> 2, 3.5 -> 4, 5 -> 4
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] + [0.0] * 24).reshape(1, 32)
    packed, _ = qz.quantize_mxfp4(ties)
    assert oracle.unpack_fp4(packed.numpy(), (32,))[:8].tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0]


def test_mxfp4_zero_block(qz):
    packed, scale = qz.quantize_mxfp4(torch.zeros(1, 64))
    assert packed.sum() == 0 and (oracle.dequant_mxfp4(packed, scale) == 0).all()


def test_fp8_quantiser(qz):
    g = torch.Generator().manual_seed(1)
    w = torch.randn(256, 256, generator=g) * 0.02
    for kind in ("e8m0", "f32"):
        q, s = qz.quantize_fp8_block128(w, kind)
        assert q.shape == (256, 256) and s.shape == (2, 2)
        if kind == "e8m0":
            deq = oracle.dequant_fp8_block128(q, s)
        else:
            deq = oracle.e4m3_to_f32(q.numpy()) * np.repeat(np.repeat(s.numpy(), 128, 0), 128, 1)
        rel = np.abs(deq - w.numpy()).max() / w.abs().max().item()
        assert rel < 0.07          # E4M3 has 3 mantissa bits: relative step 1/16
        assert not np.isnan(deq).any()


def test_expert_bank_shapes(qz):
    bank = qz.make_expert_bank(3, 64, 32, "cpu", seed=5, chunk=2)
    assert bank["w1p"].shape == (3, 32, 32) and bank["w1s"].shape == (3, 32, 2)
    assert bank["w2p"].shape == (3, 64, 16) and bank["w2s"].shape == (3, 64, 1)
    again = qz.make_expert_bank(3, 64, 32, "cpu", seed=5, chunk=2)
    assert all(torch.equal(bank[k], again[k]) for k in bank)
