"""FP8 E4M3 dense GEMV (M = 1) operator — same call as the reference's runtime/fp8_e4m3_gemv_binding.py:77-168.

    y = fp8_e4m3_gemv(W_fp8, W_scale, x, out=None, stream=None)

W_fp8 uint8 [N, K] (raw E4M3), W_scale uint8 [N/128, K/128] (E8M0, one per 128x128 tile), x bfloat16 [K].
`fp8_e4m3_gemv_f32scale` is the same with FP32 tile scales.
"""
from __future__ import annotations

from ctypes import c_int, c_int64
from typing import Optional

import torch

from . import _capi

FP8_BLOCK_TILE = 128


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _run(symbol: str, scale_dtype: torch.dtype, W_fp8, W_scale, x, out, stream):
    _require(W_fp8.is_cuda and W_scale.is_cuda and x.is_cuda, "all tensors must be on CUDA device")
    _require(W_fp8.dtype == torch.uint8, f"W_fp8 must be uint8 (raw E4M3), got {W_fp8.dtype}")
    _require(W_scale.dtype == scale_dtype, f"W_scale must be {scale_dtype}, got {W_scale.dtype}")
    _require(x.dtype == torch.bfloat16, f"x must be bfloat16, got {x.dtype}")
    _require(x.dim() == 1, f"x must be 1-D [K], got shape {tuple(x.shape)}")
    _require(W_fp8.dim() == 2, f"W_fp8 must be 2-D [N, K], got shape {tuple(W_fp8.shape)}")
    _require(W_scale.dim() == 2, f"W_scale must be 2-D [N/128, K/128], got shape {tuple(W_scale.shape)}")
    K, N = x.shape[0], W_fp8.shape[0]
    _require(W_fp8.shape[1] == K, f"W_fp8 shape {tuple(W_fp8.shape)} inconsistent with K={K}")
    _require(K % FP8_BLOCK_TILE == 0, f"K={K} must be multiple of {FP8_BLOCK_TILE}")
    _require(N % FP8_BLOCK_TILE == 0, f"N={N} must be multiple of {FP8_BLOCK_TILE}")
    want = (N // FP8_BLOCK_TILE, K // FP8_BLOCK_TILE)
    _require(tuple(W_scale.shape) == want, f"W_scale shape {tuple(W_scale.shape)} != {want}")
    if W_fp8.stride(1) != 1:
        W_fp8 = W_fp8.contiguous()
    if W_scale.stride(1) != 1:
        W_scale = W_scale.contiguous()
    x = x.contiguous()
    if out is None:
        out = torch.empty(N, dtype=torch.bfloat16, device=x.device)
    else:
        _require(tuple(out.shape) == (N,) and out.dtype == torch.bfloat16 and out.is_cuda and out.is_contiguous(),
                 f"out must be a contiguous cuda bfloat16 [{N}]")
    lib = _capi.load("fp8")
    rc = getattr(lib, symbol)(_capi.ptr(x), _capi.ptr(W_fp8), _capi.ptr(W_scale), c_int(K), c_int(N),
                              c_int64(W_fp8.stride(0) * W_fp8.element_size()),
                              c_int64(W_scale.stride(0) * W_scale.element_size()), _capi.ptr(out),
                              _capi.stream_ptr(x.device, stream))
    if rc != 0:
        raise RuntimeError(f"{symbol} returned {rc}")
    return out


def fp8_e4m3_gemv(W_fp8: torch.Tensor, W_scale: torch.Tensor, x: torch.Tensor,
                  out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    return _run("fp8_e4m3_gemv_m1", torch.uint8, W_fp8, W_scale, x, out, stream)


def fp8_e4m3_gemv_f32scale(W_fp8: torch.Tensor, W_scale: torch.Tensor, x: torch.Tensor,
                           out: Optional[torch.Tensor] = None,
                           stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    return _run("fp8_e4m3_gemv_m1_f32scale", torch.float32, W_fp8, W_scale, x, out, stream)


__all__ = ["fp8_e4m3_gemv", "fp8_e4m3_gemv_f32scale", "FP8_BLOCK_TILE"]
