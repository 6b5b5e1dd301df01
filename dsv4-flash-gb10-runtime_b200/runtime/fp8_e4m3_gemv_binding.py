"""FP8 E4M3 dense GEMV (M = 1) operator — same call as the reference's runtime/fp8_e4m3_gemv_binding.py:77-168.

    y = fp8_e4m3_gemv(W_fp8, W_scale, x, out=None, stream=None)

W_fp8 uint8 [N, K] (raw E4M3), W_scale uint8 [N/128, K/128] (E8M0, one per 128x128 tile), x bfloat16 [K].
`fp8_e4m3_gemv_f32scale` is the same with FP32 tile scales.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64
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


def fp8_e4m3_gemv_batched(W_fp8: torch.Tensor, W_scale: torch.Tensor, x: torch.Tensor, n_groups: int = 1,
                          out: Optional[torch.Tensor] = None,
                          stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Several tokens and / or several independent groups in one launch - what the reference does as a loop of
    fp8_e4m3_gemv calls, one per token (`_fp8_linear`, runtime/dsv4_engine_mxfp4.py:310-320) and one per group of the
    grouped output projection (kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:484-498):

        y[t, g*N + n] = sum_k W[g*N + n, k] * x[t, g*K + k]

    W_fp8 uint8 [n_groups*N, K], W_scale uint8 [n_groups*N/128, K/128], x bfloat16 [n_groups*K] or [S, n_groups*K];
    returns bfloat16 [n_groups*N] or [S, n_groups*N].  With one token the result equals the single-token operator's bit
    for bit; with several tokens it agrees with it to the last bfloat16 step (FP32 tensor-core sums)."""
    _require(W_fp8.is_cuda and W_scale.is_cuda and x.is_cuda, "all tensors must be on CUDA device")
    _require(W_fp8.dtype == torch.uint8, f"W_fp8 must be uint8 (raw E4M3), got {W_fp8.dtype}")
    _require(W_scale.dtype == torch.uint8, f"W_scale must be uint8 (E8M0), got {W_scale.dtype}")
    _require(x.dtype == torch.bfloat16, f"x must be bfloat16, got {x.dtype}")
    _require(x.dim() in (1, 2), f"x must be [G*K] or [S, G*K], got shape {tuple(x.shape)}")
    _require(W_fp8.dim() == 2 and W_scale.dim() == 2, "W_fp8 and W_scale must be 2-D")
    _require(n_groups >= 1, f"n_groups={n_groups} must be >= 1")
    single = x.dim() == 1
    xs = x.unsqueeze(0) if single else x
    S, K = xs.shape[0], W_fp8.shape[1]
    _require(xs.shape[1] == n_groups * K, f"x row length {xs.shape[1]} != n_groups*K = {n_groups * K}")
    _require(W_fp8.shape[0] % n_groups == 0, f"W_fp8 rows {W_fp8.shape[0]} not divisible by n_groups={n_groups}")
    N = W_fp8.shape[0] // n_groups
    _require(K % FP8_BLOCK_TILE == 0, f"K={K} must be multiple of {FP8_BLOCK_TILE}")
    _require(N % FP8_BLOCK_TILE == 0, f"N={N} must be multiple of {FP8_BLOCK_TILE}")
    want = (n_groups * N // FP8_BLOCK_TILE, K // FP8_BLOCK_TILE)
    _require(tuple(W_scale.shape) == want, f"W_scale shape {tuple(W_scale.shape)} != {want}")
    if W_fp8.stride(1) != 1:
        W_fp8 = W_fp8.contiguous()
    if W_scale.stride(1) != 1:
        W_scale = W_scale.contiguous()
    if xs.stride(1) != 1:
        xs = xs.contiguous()
    if out is None:
        out2 = torch.empty(S, n_groups * N, dtype=torch.bfloat16, device=x.device)
    else:
        shape = (n_groups * N,) if single else (S, n_groups * N)
        _require(tuple(out.shape) == shape and out.dtype == torch.bfloat16 and out.is_cuda and out.stride(-1) == 1,
                 f"out must be a cuda bfloat16 {list(shape)} with unit inner stride")
        out2 = out.unsqueeze(0) if single else out
    lib = _capi.load("fp8")
    rc = lib.fp8_e4m3_gemv_batched(_capi.ptr(xs), _capi.ptr(W_fp8), _capi.ptr(W_scale), c_int(K), c_int(N),
                                   c_int64(W_fp8.stride(0)), c_int64(W_scale.stride(0)), c_int(n_groups), c_int(S),
                                   c_int64(xs.stride(0) if S > 1 else n_groups * K),
                                   c_int64(out2.stride(0) if S > 1 else n_groups * N), _capi.ptr(out2),
                                   _capi.stream_ptr(x.device, stream))
    if rc != 0:
        raise RuntimeError(f"fp8_e4m3_gemv_batched returned {rc}")
    return out2[0] if single else out2


def fp8_shared_swiglu(shared: dict, x: torch.Tensor, limit_gate: float = 10.0, limit_up: float = 0.0,
                      out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                      stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """The shared expert's gated FFN for one token (reference: three fp8 GEMVs and an activation kernel,
    kernel/cpp-engine-mxfp4/dsv4_engine_mxfp4_wire.cu:523-556): out = W2 (silu(clamp(W1 x)) * clamp(W3 x)).

    `shared`: w1, w3 uint8 [hidden, K] and w2 uint8 [out_dim, hidden] raw E4M3, w1s / w3s / w2s uint8 E8M0 tile scales
    (what bank_loader.load_shared_expert_fp8 returns); x bfloat16 [K].  The defaults are the C++ engine's clamp (gate
    only, 10); the Python engine clamps both (10, 10)."""
    w1, w3, w2 = shared["w1"], shared["w3"], shared["w2"]
    K, hidden, out_dim = x.numel(), w1.shape[0], w2.shape[0]
    for name, t in (("w1", w1), ("w3", w3), ("w2", w2), ("w1s", shared["w1s"]), ("w3s", shared["w3s"]), ("w2s", shared["w2s"])):
        _require(t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous(), f"{name} must be a contiguous cuda uint8 tensor")
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 1 and x.is_contiguous(), "x must be a contiguous cuda bfloat16 [K]")
    _require(tuple(w1.shape) == (hidden, K) and tuple(w3.shape) == (hidden, K) and tuple(w2.shape) == (out_dim, hidden),
             "w1 / w3 must be [hidden, K] and w2 [out_dim, hidden]")
    for name, t, rows, cols in (("w1s", shared["w1s"], hidden, K), ("w3s", shared["w3s"], hidden, K), ("w2s", shared["w2s"], out_dim, hidden)):
        _require(tuple(t.shape) == (rows // FP8_BLOCK_TILE, cols // FP8_BLOCK_TILE), f"{name} must be [{rows}/128, {cols}/128]")
    lib = _capi.load("fp8")
    need = lib.fp8_e4m3_shared_swiglu_workspace_bytes(c_int(hidden))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    _require(workspace.is_cuda and workspace.numel() * workspace.element_size() >= need, f"workspace needs {need} bytes")
    if out is None:
        out = torch.empty(out_dim, dtype=torch.bfloat16, device=x.device)
    _require(tuple(out.shape) == (out_dim,) and out.dtype == torch.bfloat16 and out.is_cuda and out.is_contiguous(),
             f"out must be a contiguous cuda bfloat16 [{out_dim}]")
    rc = lib.fp8_e4m3_shared_swiglu_m1(_capi.ptr(x), _capi.ptr(w1), _capi.ptr(shared["w1s"]), _capi.ptr(w3),
                                       _capi.ptr(shared["w3s"]), _capi.ptr(w2), _capi.ptr(shared["w2s"]), c_int(K),
                                       c_int(hidden), c_int(out_dim), c_float(limit_gate), c_float(limit_up),
                                       _capi.ptr(out), _capi.ptr(workspace), _capi.stream_ptr(x.device, stream))
    if rc != 0:
        raise RuntimeError(f"fp8_e4m3_shared_swiglu_m1 returned {rc}")
    return out


__all__ = ["fp8_e4m3_gemv", "fp8_e4m3_gemv_f32scale", "fp8_e4m3_gemv_batched", "fp8_shared_swiglu", "FP8_BLOCK_TILE"]
