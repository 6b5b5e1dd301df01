"""Synthetic-weight quantisers: float -> MXFP4 (E2M1 + E8M0 per 32) and float -> FP8 E4M3 with 128x128 scales.

The reference ships no quantiser (its weights arrive pre-quantised), so these follow the rule the benchmark
configurations state:

  MXFP4: per 32 contiguous K elements, e = floor(log2(amax)) - 2, scale byte = e + 127 (clamped to 0..254),
         element = w / 2^e rounded to the nearest E2M1 value (ties to the even code), saturated at +-6;
         two elements per byte, low nibble = even k.
  FP8:   per 128x128 block, scale = amax / 448 (FP32) or the next power of two above it (E8M0 byte),
         element = w / scale rounded to nearest E4M3.

Pure torch; runs on CPU or CUDA tensors.  Used to build benchmark and test inputs, never on the kernel path.
"""
from __future__ import annotations

import torch

MXFP4_BLOCK = 32
FP8_TILE = 128
E4M3_MAX = 448.0


def _floor_log2(a: torch.Tensor) -> torch.Tensor:
    """floor(log2(a)) for positive finite float32 a, exact (from the exponent field)."""
    _, ex = torch.frexp(a.float())          # a = m * 2^ex, m in [0.5, 1)
    return ex.to(torch.int32) - 1


def quantize_mxfp4(w: torch.Tensor):
    """w [..., K] float -> (packed uint8 [..., K/2], scale uint8 [..., K/32])."""
    if w.shape[-1] % MXFP4_BLOCK:
        raise ValueError(f"last dim {w.shape[-1]} is not a multiple of {MXFP4_BLOCK}")
    wf = w.float()
    blocks = wf.reshape(*wf.shape[:-1], -1, MXFP4_BLOCK)
    amax = blocks.abs().amax(dim=-1)
    e = torch.where(amax > 0, _floor_log2(torch.where(amax > 0, amax, torch.ones_like(amax))) - 2,
                    torch.full_like(amax, -127, dtype=torch.int32))
    e = e.clamp(-127, 127)
    scale_byte = (e + 127).to(torch.uint8)
    q = torch.ldexp(blocks, (-e).unsqueeze(-1).expand_as(blocks))
    a = q.abs()
    # E2M1 magnitudes 0 .5 1 1.5 2 3 4 6 -> codes 0..7; midpoints go to the even code
    code = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
            + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
            + (a > 5.0).to(torch.uint8))
    code = code | (torch.signbit(q).to(torch.uint8) << 3)
    code = code.reshape(*wf.shape)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), scale_byte.contiguous()


def quantize_fp8_block128(w: torch.Tensor, scale_kind: str = "e8m0"):
    """w [N, K] float -> (bytes uint8 [N, K], scale [N/128, K/128]).

    scale_kind 'e8m0': uint8 scale bytes, 2^ceil(log2(amax/448)); 'f32': float32 scale amax/448.
    """
    n, k = w.shape
    if n % FP8_TILE or k % FP8_TILE:
        raise ValueError(f"shape {tuple(w.shape)} is not a multiple of {FP8_TILE}")
    wf = w.float()
    tiles = wf.reshape(n // FP8_TILE, FP8_TILE, k // FP8_TILE, FP8_TILE)
    amax = tiles.abs().amax(dim=(1, 3))
    s = amax / E4M3_MAX
    s = torch.where(s > 0, s, torch.ones_like(s))
    if scale_kind == "e8m0":
        m, ex = torch.frexp(s)                          # s = m * 2^ex, m in [0.5, 1)
        e = torch.where(m == 0.5, ex - 1, ex).to(torch.int32).clamp(-127, 127)   # ceil(log2 s)
        scale_out = (e + 127).to(torch.uint8)
        s_used = torch.ldexp(torch.ones_like(s), e)
    elif scale_kind == "f32":
        scale_out = s.contiguous()
        s_used = s
    else:
        raise ValueError("scale_kind must be 'e8m0' or 'f32'")
    q = (tiles / s_used[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).reshape(n, k)
    return q.to(torch.float8_e4m3fn).view(torch.uint8).contiguous(), scale_out.contiguous()


def make_expert_bank(n_experts: int, hidden: int, ff: int, device, seed: int, std: float = 0.02,
                     chunk: int = 8):
    """Random N(0, std) experts quantised to MXFP4: dict of w1p/w3p [E, ff, hidden/2], w2p [E, hidden, ff/2]
    and their E8M0 scales, generated `chunk` experts at a time so the float copy stays small."""
    gen = torch.Generator(device=device).manual_seed(seed)
    bank = {
        "w1p": torch.empty(n_experts, ff, hidden // 2, dtype=torch.uint8, device=device),
        "w3p": torch.empty(n_experts, ff, hidden // 2, dtype=torch.uint8, device=device),
        "w2p": torch.empty(n_experts, hidden, ff // 2, dtype=torch.uint8, device=device),
        "w1s": torch.empty(n_experts, ff, hidden // 32, dtype=torch.uint8, device=device),
        "w3s": torch.empty(n_experts, ff, hidden // 32, dtype=torch.uint8, device=device),
        "w2s": torch.empty(n_experts, hidden, ff // 32, dtype=torch.uint8, device=device),
    }
    for e0 in range(0, n_experts, chunk):
        e1 = min(n_experts, e0 + chunk)
        for key, shape in (("w1", (e1 - e0, ff, hidden)), ("w3", (e1 - e0, ff, hidden)), ("w2", (e1 - e0, hidden, ff))):
            w = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std
            p, s = quantize_mxfp4(w.to(torch.bfloat16))
            bank[key + "p"][e0:e1] = p
            bank[key + "s"][e0:e1] = s
    return bank


__all__ = ["quantize_mxfp4", "quantize_fp8_block128", "make_expert_bank", "MXFP4_BLOCK", "FP8_TILE"]
