"""CPU restatement of the reference's quantized-weight path (TEST INFRASTRUCTURE).

Every function names the reference location whose behaviour it restates
(paths are relative to the reference project's root).  Arithmetic is numpy on
bytes / float32; torch is used only to round to bfloat16 and for the FP32
matmul, as the reference's own ground-truth path does
(runtime/mxfp4_loader.py:292-305 then a torch matmul).
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = [
    "FP4_E2M1_VALUES", "unpack_fp4", "pack_fp4", "e8m0_to_f32", "e4m3_to_f32",
    "dequant_mxfp4", "dequant_fp8_block128", "bf16_round", "bf16_bits",
    "mxfp4_gemv_ref", "fp8_gemv_ref", "shared_swiglu_fp8_ref", "grouped_gemv_ref", "moe_layer_ref",
    "router_scores_sqrt_softplus", "topk_lowest_index", "route_sqrt_softplus",
    "route_softmax", "max_abs_rel", "cosine", "MXFP4_BLOCK", "FP8_TILE",
]

MXFP4_BLOCK = 32     # elements per E8M0 scale (runtime/mxfp4_loader.py:96)
FP8_TILE = 128       # FP8 weights carry one E8M0 byte per 128x128 tile (runtime/fp8_e4m3_gemv_binding.py:25)

# E2M1 codebook indexed by the raw nibble (runtime/mxfp4_unpack.py:36-39,
# kernel/mxfp4-dense/mxfp4_gemv.cu:57-60, kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:66-69).
FP4_E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


# --------------------------------------------------------------------------- formats

def unpack_fp4(packed, shape=None) -> np.ndarray:
    """Bytes -> codebook values, no scale (runtime/mxfp4_unpack.py:47-118).

    The low nibble of byte i is element 2i, the high nibble element 2i+1
    (runtime/mxfp4_unpack.py:18-23, :106-112).  Returns float32.
    """
    b = np.ascontiguousarray(_as_u8(packed)).reshape(-1)
    out = np.empty(b.size * 2, dtype=np.float32)
    out[0::2] = FP4_E2M1_VALUES[b & 0x0F]
    out[1::2] = FP4_E2M1_VALUES[b >> 4]
    if shape is None:
        src = _as_u8(packed).shape
        shape = tuple(src[:-1]) + (src[-1] * 2,)
    if int(np.prod(shape)) != out.size:
        raise ValueError(f"{b.size} bytes hold {out.size} nibbles, shape {shape} wants {int(np.prod(shape))}")
    return out.reshape(shape)


def pack_fp4(values) -> np.ndarray:
    """Codebook values -> bytes, inverse of unpack_fp4 (runtime/mxfp4_unpack.py:121-168).

    -0.0 maps to nibble 8 and +0.0 to nibble 0; any value outside the codebook
    raises ValueError, like the reference.
    """
    v = np.ascontiguousarray(_as_f32(values)).reshape(-1)
    if v.size % 2:
        raise ValueError(f"element count must be even, got {v.size}")
    mag = np.abs(v)
    idx = np.full(v.size, 255, dtype=np.uint8)
    for code in range(8):
        idx[mag == FP4_E2M1_VALUES[code]] = code
    if (idx == 255).any():
        bad = int(np.flatnonzero(idx == 255)[0])
        raise ValueError(f"value {v[bad]} at index {bad} is not an E2M1 value")
    idx |= (np.signbit(v).astype(np.uint8) << 3)
    return (idx[0::2] | (idx[1::2] << 4)).astype(np.uint8)


def e8m0_to_f32(scale_bytes, ff: str = "nan") -> np.ndarray:
    """E8M0 byte -> 2^(b-127) as float32 (runtime/e8m0_decode.py:32-64).

    Byte 0 gives the float32 subnormal 2^-127, byte 127 gives 1.0.  Byte 0xFF is
    NaN in the reference's Python (`ff="nan"`, runtime/e8m0_decode.py:57-63) and
    0.0 in all three reference CUDA kernels (`ff="zero"`,
    kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:74-78, kernel/mxfp4-dense/mxfp4_gemv.cu:65-69,
    kernel/fp8-dense/fp8_e4m3_gemv.cu:58-62).
    """
    b = _as_u8(scale_bytes)
    with np.errstate(over="ignore"):   # byte 255 -> 2^128 overflows to inf before it is replaced below
        out = np.ldexp(np.float64(1.0), b.astype(np.int32) - 127).astype(np.float32)
    if ff == "nan":
        out = np.where(b == 0xFF, np.float32(np.nan), out)
    elif ff == "zero":
        out = np.where(b == 0xFF, np.float32(0.0), out)
    else:
        raise ValueError("ff must be 'nan' or 'zero'")
    return out.astype(np.float32)


def _e4m3_table() -> np.ndarray:
    # OCP FP8 E4M3 ("fn": no infinities, S.1111.111 is NaN), bias 7: the values
    # torch's float8_e4m3fn view yields at runtime/dsv4_engine_mxfp4.py:539-541.
    t = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


_E4M3 = _e4m3_table()


def e4m3_to_f32(w_bytes) -> np.ndarray:
    """Raw E4M3 bytes -> float32 (runtime/dsv4_engine_mxfp4.py:539-541)."""
    return _E4M3[_as_u8(w_bytes)]


def bf16_round(x) -> torch.Tensor:
    """float32 -> bfloat16, round-to-nearest-even, as `.to(torch.bfloat16)` does."""
    return torch.from_numpy(np.ascontiguousarray(_as_f32(x))).to(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    """bfloat16 tensor -> its int16 bit patterns (so that -0.0 != +0.0 in comparisons)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy()


# --------------------------------------------------------------------------- dequantisation

def dequant_mxfp4(packed, scale, ff: str = "nan") -> np.ndarray:
    """[rows, cols/2] bytes + [rows, cols/32] E8M0 -> float32 [rows, cols].

    Restates MXFP4Loader.dequant_mxfp4 (runtime/mxfp4_loader.py:272-309): unpack,
    view as [rows, cols/32, 32], multiply by the decoded scale.  Every product
    is exact in bfloat16, so bf16_round() of the result is the reference's output.
    """
    p = _as_u8(packed)
    s = _as_u8(scale)
    rows, half = p.shape
    cols = half * 2
    if s.shape != (rows, cols // MXFP4_BLOCK):
        raise ValueError(f"scale shape {s.shape} != ({rows}, {cols // MXFP4_BLOCK})")
    vals = unpack_fp4(p, (rows, cols // MXFP4_BLOCK, MXFP4_BLOCK))
    with np.errstate(over="ignore", invalid="ignore"):
        return (vals * e8m0_to_f32(s, ff)[..., None]).reshape(rows, cols)


def dequant_fp8_block128(w_bytes, scale_bytes, ff: str = "nan") -> np.ndarray:
    """[N, K] E4M3 bytes + [N/128, K/128] E8M0 -> float32 [N, K].

    Restates _fp8_dequant_to_bf16 (runtime/dsv4_engine_mxfp4.py:531-553): the
    scale is repeated 128x along both axes and multiplied in.
    """
    w = e4m3_to_f32(w_bytes)
    n, k = w.shape
    s = e8m0_to_f32(scale_bytes, ff)
    s_full = np.repeat(np.repeat(s, FP8_TILE, axis=0), FP8_TILE, axis=1)[:n, :k]
    with np.errstate(over="ignore", invalid="ignore"):
        return w * s_full


# --------------------------------------------------------------------------- GEMV / MoE

def _matvec(w_f32: np.ndarray, x_f32: np.ndarray) -> np.ndarray:
    return torch.mv(torch.from_numpy(np.ascontiguousarray(w_f32)),
                    torch.from_numpy(np.ascontiguousarray(x_f32))).numpy()


def mxfp4_gemv_ref(packed, scale, x_bf16: torch.Tensor) -> np.ndarray:
    """y[n] = sum_k W[n,k] x[k] in FP32 (kernel/mxfp4-dense/mxfp4_gemv.cu:72-128).

    Scale byte 0xFF contributes 0 as in the kernel.  Returns float32 (before the
    final bf16 rounding the kernel applies at :127).
    """
    return _matvec(dequant_mxfp4(packed, scale, ff="zero"), x_bf16.float().numpy())


def fp8_gemv_ref(w_bytes, scale_bytes, x_bf16: torch.Tensor) -> np.ndarray:
    """y[n] = sum_k e4m3(W[n,k]) 2^(S[n/128,k/128]-127) x[k] (kernel/fp8-dense/fp8_e4m3_gemv.cu:74-129)."""
    return _matvec(dequant_fp8_block128(w_bytes, scale_bytes, ff="zero"), x_bf16.float().numpy())


def _silu(v: np.ndarray) -> np.ndarray:
    v = v.astype(np.float32)
    with np.errstate(over="ignore"):      # exp(+large) -> inf -> v / inf = -0.0, the right limit
        return v / (1.0 + np.exp(-v, dtype=np.float32))


def shared_swiglu_fp8_ref(x_bf16: torch.Tensor, shared: dict, limit_gate: float = 10.0, limit_up: float = 0.0) -> np.ndarray:
    """The shared expert's FP8 gated FFN for one token, FP32 throughout:
    out = W2 (silu(clamp(W1 x, +-limit_gate)) * clamp(W3 x, +-limit_up)), a limit <= 0 meaning no clamp.

    Restates runtime/dsv4_engine_mxfp4.py:399-410 (clamps both, limit 10) and
    kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:506-556 (clamps the gate only); both round every GEMV output
    and the activation to bf16, the oracle keeps FP32 (the tolerance is stated against it).  `shared`: w1, w3
    [hidden, K], w2 [O, hidden] raw E4M3 bytes, w1s / w3s / w2s E8M0 128x128 tile scales.  Returns float32 [O].
    """
    x = x_bf16.float().numpy()
    g = _matvec(dequant_fp8_block128(shared["w1"], shared["w1s"], ff="zero"), x)
    u = _matvec(dequant_fp8_block128(shared["w3"], shared["w3s"], ff="zero"), x)
    if limit_gate > 0:
        g = np.clip(g, -limit_gate, limit_gate)
    if limit_up > 0:
        u = np.clip(u, -limit_up, limit_up)
    return _matvec(dequant_fp8_block128(shared["w2"], shared["w2s"], ff="zero"), (_silu(g) * u).astype(np.float32))


def grouped_gemv_ref(x_bf16, w1p, w3p, w2p, w1s, w3s, w2s, r) -> np.ndarray:
    """out = sum_e r[e] * W2_e (silu(W1_e x) * (W3_e x)), FP32 throughout.

    Restates kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:9-14 (no SwiGLU clamp on
    the routed path).  The reference kernel rounds the intermediate to bf16
    (:208); the oracle keeps FP32, which is the FP32 reference the tolerance
    is stated against.  Inputs are stacked per expert: w1p/w3p [E, H, K/2],
    w2p [E, O, H/2], scales likewise.  Returns float32 [O].
    """
    x = x_bf16.float().numpy()
    r = _as_f32(r)
    out = None
    for e in range(_as_u8(w1p).shape[0]):
        g = _matvec(dequant_mxfp4(w1p[e], w1s[e], "zero"), x)
        u = _matvec(dequant_mxfp4(w3p[e], w3s[e], "zero"), x)
        m = _silu(g) * u
        y = _matvec(dequant_mxfp4(w2p[e], w2s[e], "zero"), m)
        out = r[e] * y if out is None else out + r[e] * y
    return out.astype(np.float32)


def moe_layer_ref(x_bf16: torch.Tensor, bank: dict, ids, w) -> np.ndarray:
    """Routed MoE over T tokens: out[t] = sum_j w[t,j] * FFN_{ids[t,j]}(x[t]).

    `bank` holds w1p/w3p [E, H, K/2], w2p [E, O, H/2] and w1s/w3s/w2s for all E
    experts.  Each distinct expert is dequantised once and applied to all of its
    tokens with one FP32 matmul (same arithmetic as
    runtime/dsv4_engine_mxfp4.py:412-422, which loops tokens one by one).
    """
    x = x_bf16.float().numpy()
    ids = np.asarray(ids)
    w = _as_f32(w)
    t_count = x.shape[0]
    out = np.zeros((t_count, _as_u8(bank["w2p"]).shape[1]), dtype=np.float32)
    for e in np.unique(ids):
        tok, slot = np.nonzero(ids == e)
        w1 = torch.from_numpy(dequant_mxfp4(bank["w1p"][e], bank["w1s"][e], "zero"))
        w3 = torch.from_numpy(dequant_mxfp4(bank["w3p"][e], bank["w3s"][e], "zero"))
        w2 = torch.from_numpy(dequant_mxfp4(bank["w2p"][e], bank["w2s"][e], "zero"))
        xe = torch.from_numpy(x[tok])
        g = (xe @ w1.T).numpy()
        u = (xe @ w3.T).numpy()
        m = torch.from_numpy(_silu(g) * u)
        y = (m @ w2.T).numpy()
        # a token lists an expert at most once, so tok has no duplicates here
        out[tok] += w[tok, slot][:, None] * y
    return out


# --------------------------------------------------------------------------- routing

def router_scores_sqrt_softplus(logits) -> np.ndarray:
    """score = sqrt(softplus(logit)) in float32 (kernel/cpp-engine-mxfp4/routed.cu:156-164)."""
    g = _as_f32(logits)
    sp = np.maximum(g, np.float32(0)) + np.log1p(np.exp(-np.abs(g), dtype=np.float32), dtype=np.float32)
    return np.sqrt(sp, dtype=np.float32)


def topk_lowest_index(scores, k: int):
    """k largest scores per row, descending, ties to the lowest index.

    Restates the strict `>` scan of topk6_norm_scale_host
    (kernel/cpp-engine-mxfp4/routed.cu:183-199).
    """
    s = np.atleast_2d(_as_f32(scores))
    order = np.argsort(-s, axis=-1, kind="stable")[:, :k]
    return order.astype(np.int32), np.take_along_axis(s, order, axis=-1)


def route_sqrt_softplus(logits, k: int = 6, scaling: float = 1.5, eps: float = 1e-20):
    """Reference routing: sqrt-softplus scores, top-k, w = s / (sum s + eps) * scaling.

    Normalisation is done in float64 and rounded to float32 like the engine
    (kernel/cpp-engine-mxfp4/routed.cu:200-206); the Python twin is
    runtime/dsv4_engine_mxfp4.py:363-370.
    """
    ids, top = topk_lowest_index(router_scores_sqrt_softplus(logits), k)
    denom = top.astype(np.float64).sum(-1, keepdims=True) + eps
    w = (top.astype(np.float64) / denom * scaling).astype(np.float32)
    return ids, w


def route_softmax(logits, k: int = 6):
    """Softmax over all experts, top-k, weights renormalised to sum 1.

    This is the routing rule the benchmark configurations state; selection is the
    same as route_sqrt_softplus because both scores grow with the logit.
    """
    g = np.atleast_2d(_as_f32(logits)).astype(np.float64)
    p = np.exp(g - g.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    ids, _ = topk_lowest_index(np.atleast_2d(_as_f32(logits)), k)
    top = np.take_along_axis(p, ids.astype(np.int64), axis=-1)
    w = (top / top.sum(-1, keepdims=True)).astype(np.float32)
    return ids, w


# --------------------------------------------------------------------------- metrics

def max_abs_rel(out, ref) -> float:
    """max|out-ref| / max|ref| : the quantity bounded by 1e-2 in the acceptance rule."""
    o = _as_f32(out).astype(np.float64)
    r = _as_f32(ref).astype(np.float64)
    denom = np.abs(r).max()
    return float(np.abs(o - r).max() / (denom if denom > 0 else 1.0))


def cosine(out, ref) -> float:
    o = _as_f32(out).astype(np.float64).reshape(-1)
    r = _as_f32(ref).astype(np.float64).reshape(-1)
    d = np.linalg.norm(o) * np.linalg.norm(r)
    return float(o @ r / d) if d > 0 else 1.0


# --------------------------------------------------------------------------- helpers

def _as_u8(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().contiguous()
        if a.dtype not in (torch.uint8, torch.int8):
            raise TypeError(f"expected 8-bit tensor, got {a.dtype}")
        return a.view(torch.uint8).numpy()
    a = np.asarray(a)
    if a.dtype == np.int8:
        return a.view(np.uint8)
    if a.dtype != np.uint8:
        raise TypeError(f"expected uint8, got {a.dtype}")
    return a


def _as_f32(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        return a.detach().cpu().float().numpy()
    return np.asarray(a, dtype=np.float32)
