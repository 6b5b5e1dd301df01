"""The CPU oracle against vectors produced by the reference's own Python modules (tests/golden/make_golden.py)."""
import numpy as np
import torch

import oracle


def test_fp4_unpack_every_byte(golden):
    got = oracle.unpack_fp4(golden["fp4_all_bytes_in"], (512,))
    assert np.array_equal(got.view(np.uint32), golden["fp4_all_bytes_out_bits"])   # bit patterns: -0.0 kept


def test_fp4_pack_is_the_inverse(golden):
    vals = golden["fp4_all_bytes_out_bits"].view(np.float32)
    assert np.array_equal(oracle.pack_fp4(vals), golden["fp4_pack_roundtrip"])
    assert np.array_equal(oracle.pack_fp4(vals), golden["fp4_all_bytes_in"])


def test_e8m0_every_byte(golden):
    got = oracle.e8m0_to_f32(np.arange(256, dtype=np.uint8), ff="nan")
    ref = golden["e8m0_all_bytes_bits"].view(np.float32)
    assert np.isnan(got[255]) and np.isnan(ref[255])
    assert np.array_equal(got[:255].view(np.uint32), golden["e8m0_all_bytes_bits"][:255])
    assert np.array_equal(golden["e8m0_all_bytes_bits"][:255], golden["e8m0_all_bytes_torch_bits"][:255])
    # known answers stated in the reference's docstring
    assert got[127] == 1.0 and got[0] == np.float32(2.0 ** -127) and got[254] == np.float32(2.0 ** 127)
    assert oracle.e8m0_to_f32(np.array([255], np.uint8), ff="zero")[0] == 0.0


def test_e4m3_every_byte(golden):
    got = oracle.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    ref = golden["e4m3_all_bytes_bits"].view(np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan) and nan.sum() == 2
    assert np.array_equal(got[~nan].view(np.uint32), golden["e4m3_all_bytes_bits"][~nan])


def _same_bf16(bits_a, bits_b):
    a = torch.from_numpy(np.ascontiguousarray(bits_a)).view(torch.bfloat16).float().numpy()
    b = torch.from_numpy(np.ascontiguousarray(bits_b)).view(torch.bfloat16).float().numpy()
    nan = np.isnan(a)
    return np.array_equal(nan, np.isnan(b)) and np.array_equal(bits_a[~nan], bits_b[~nan])


def test_mxfp4_dequant_matches_reference_loader(golden):
    deq = oracle.dequant_mxfp4(golden["mxfp4_packed"], golden["mxfp4_scale"], ff="nan")
    got = oracle.bf16_bits(oracle.bf16_round(deq))
    assert _same_bf16(got, golden["mxfp4_dequant_bf16_bits"])
    # the block with scale 0xFF is NaN in the loader and 0 in kernel semantics
    assert np.isnan(deq[0, 96:128]).all()
    assert (oracle.dequant_mxfp4(golden["mxfp4_packed"], golden["mxfp4_scale"], ff="zero")[0, 96:128] == 0).all()


def test_fp8_dequant_matches_reference_engine(golden):
    deq = oracle.dequant_fp8_block128(golden["fp8_bytes"], golden["fp8_scale"], ff="nan")
    got = oracle.bf16_bits(oracle.bf16_round(deq))
    assert _same_bf16(got, golden["fp8_dequant_bf16_bits"])


def test_router_matches_reference_route(golden):
    logits = golden["route_logits"]
    scores = oracle.router_scores_sqrt_softplus(logits)
    ref_scores = golden["route_scores_bits"].view(np.float32)
    # numpy and torch may differ in the last bit of log1p/exp; selection below is checked on the reference scores
    np.testing.assert_allclose(scores, ref_scores, rtol=3e-7, atol=1e-22)   # atol: subnormal softplus(-100)
    ids, w = oracle.route_sqrt_softplus(logits)
    ref_ids = golden["route_ids"]
    ref_w = torch.from_numpy(golden["route_w_bf16_bits"]).view(torch.bfloat16).float().numpy()
    for t in range(logits.shape[0]):
        # same scores picked, in the same (descending) order; on exact ties the engine takes the lowest index
        assert np.array_equal(ref_scores[t][ids[t]], ref_scores[t][ref_ids[t]])
        if len(np.unique(ref_scores[t])) == ref_scores.shape[1]:
            assert np.array_equal(ids[t], ref_ids[t])
        got_w = torch.from_numpy(w[t]).to(torch.bfloat16).float().numpy()
        np.testing.assert_allclose(got_w, ref_w[t], rtol=2 ** -7, atol=1e-20)   # atol: weights from subnormal scores
    # tie rule of the C++ engine: strict '>' scan keeps the lowest index
    tie_ids, _ = oracle.topk_lowest_index(np.array([[1.0, 3.0, 3.0, 2.0, 3.0]], np.float32), 3)
    assert tie_ids.tolist() == [[1, 2, 4]]


def test_softmax_route_selects_like_sqrt_softplus():
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((16, 256)).astype(np.float32)
    ids_a, w_a = oracle.route_softmax(logits)
    ids_b, _ = oracle.route_sqrt_softplus(logits)
    assert np.array_equal(ids_a, ids_b)
    np.testing.assert_allclose(w_a.sum(-1), 1.0, rtol=1e-6)


def test_expert_byte_count():
    # bytes of one routed expert as the reference counts them (tools/D27_baseline.py:60)
    k, ff = 4096, 2048
    per_expert = 2 * (ff * k // 2 + ff * k // 32) + (k * ff // 2 + k * ff // 32)
    assert per_expert == 13369344
