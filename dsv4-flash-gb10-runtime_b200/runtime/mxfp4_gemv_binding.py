"""MXFP4 dense GEMV (M = 1) operator — same call as the reference's runtime/mxfp4_gemv_binding.py:67-154.

    y = mxfp4_gemv(W_packed, W_scale, x, out=None, stream=None)

W_packed uint8 [N, K/2] (low nibble = even k), W_scale uint8 [N, K/32] (E8M0), x bfloat16 [K]; all CUDA.
Returns bfloat16 [N].  Raises RuntimeError on a shape / dtype / device mismatch or a non-zero return code.
"""
from __future__ import annotations

from ctypes import c_int, c_int64
from typing import Optional

import torch

from . import _capi


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def mxfp4_gemv(W_packed: torch.Tensor, W_scale: torch.Tensor, x: torch.Tensor,
               out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    _require(W_packed.is_cuda and W_scale.is_cuda and x.is_cuda, "all tensors must be on CUDA device")
    _require(W_packed.dtype == torch.uint8, f"W_packed must be uint8, got {W_packed.dtype}")
    _require(W_scale.dtype == torch.uint8, f"W_scale must be uint8, got {W_scale.dtype}")
    _require(x.dtype == torch.bfloat16, f"x must be bfloat16, got {x.dtype}")
    _require(x.dim() == 1, f"x must be 1-D [K], got shape {tuple(x.shape)}")
    _require(W_packed.dim() == 2, f"W_packed must be 2-D [N, K/2], got shape {tuple(W_packed.shape)}")
    _require(W_scale.dim() == 2, f"W_scale must be 2-D [N, K/32], got shape {tuple(W_scale.shape)}")
    K, N = x.shape[0], W_packed.shape[0]
    _require(K % 32 == 0, f"K={K} must be multiple of 32")
    _require(W_packed.shape[1] == K // 2, f"W_packed shape {tuple(W_packed.shape)} inconsistent with K={K}")
    _require(tuple(W_scale.shape) == (N, K // 32), f"W_scale shape {tuple(W_scale.shape)} != ({N}, {K // 32})")
    # rows may be strided (a slice of a larger matrix); only the last axis must be dense
    if W_packed.stride(1) != 1:
        W_packed = W_packed.contiguous()
    if W_scale.stride(1) != 1:
        W_scale = W_scale.contiguous()
    x = x.contiguous()
    if out is None:
        out = torch.empty(N, dtype=torch.bfloat16, device=x.device)
    else:
        _require(tuple(out.shape) == (N,) and out.dtype == torch.bfloat16 and out.is_cuda and out.is_contiguous(),
                 f"out must be a contiguous cuda bfloat16 [{N}]")
    lib = _capi.load("mxfp4")
    rc = lib.mxfp4_gemv_m1(_capi.ptr(x), _capi.ptr(W_packed), _capi.ptr(W_scale), c_int(K), c_int(N),
                           c_int64(W_packed.stride(0)), c_int64(W_scale.stride(0)), _capi.ptr(out),
                           _capi.stream_ptr(x.device, stream))
    if rc != 0:
        raise RuntimeError(f"mxfp4_gemv_m1 returned {rc}")
    return out


__all__ = ["mxfp4_gemv"]
