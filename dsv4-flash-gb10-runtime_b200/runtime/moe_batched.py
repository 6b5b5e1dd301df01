"""Routed-expert MoE layer for a batch of tokens (batched decode, prefill) on the tcgen05 tensor cores.

    out = moe_forward(bank, x, ids, weights)

bank: dict of 'w1p','w3p' uint8 [E, hidden, K/2], 'w2p' [E, out_dim, hidden/2] and the E8M0 scales 'w1s','w3s','w2s';
x bfloat16 [T, K]; ids int32 [T, k] (a token lists an expert at most once); weights float32 [T, k].
Returns bfloat16 [T, out_dim].  The reference has no batched path (it loops tokens,
runtime/dsv4_engine_mxfp4.py:412-422); the result is the same per-token FFN sum.
"""
from __future__ import annotations

from ctypes import c_int
from typing import Dict, Optional

import torch

from . import _capi


def forward_workspace_bytes(n_tokens: int, k: int, K_in: int, hidden: int, out_dim: int, n_experts: int) -> int:
    return int(_capi.load("moe").mxfp4_moe_forward_workspace_bytes(n_tokens, k, K_in, hidden, out_dim, n_experts))


def moe_forward(bank: Dict[str, torch.Tensor], x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                path: Optional[str] = None) -> torch.Tensor:
    """`path`: None = the library's default (block-scaled MXFP4 MMAs unless DSV4_B200_MOE_PATH=fp16), 'mxf4' =
    block-scaled MMAs fed with the packed weights (activations as three MXFP4 terms), 'fp16' = fp16 MMAs with
    in-kernel dequantisation (exact operands)."""
    lib = _capi.load("moe")
    for name, t, dt in (("x", x, torch.bfloat16), ("ids", ids, torch.int32), ("weights", weights, torch.float32)):
        if not t.is_cuda or t.dtype != dt or not t.is_contiguous():
            raise ValueError(f"{name}: expected a contiguous CUDA tensor of {dt}")
    T, K = x.shape
    k = ids.shape[1]
    E, hidden, out_dim = bank["w1p"].shape[0], bank["w1p"].shape[1], bank["w2p"].shape[1]
    if tuple(ids.shape) != (T, k) or tuple(weights.shape) != (T, k):
        raise ValueError("ids / weights must be [T, k]")
    if bank["w1p"].shape[2] != K // 2 or bank["w2p"].shape[2] != hidden // 2:
        raise ValueError("bank shapes do not match x")
    if out is None:
        out = torch.empty(T, out_dim, dtype=torch.bfloat16, device=x.device)
    if workspace is None:
        workspace = torch.empty(forward_workspace_bytes(T, k, K, hidden, out_dim, E), dtype=torch.uint8, device=x.device)
    args = (_capi.ptr(x), _capi.ptr(bank["w1p"]), _capi.ptr(bank["w3p"]), _capi.ptr(bank["w2p"]),
                               _capi.ptr(bank["w1s"]), _capi.ptr(bank["w3s"]), _capi.ptr(bank["w2s"]), _capi.ptr(ids),
                               _capi.ptr(weights), c_int(T), c_int(E), c_int(K), c_int(hidden), c_int(out_dim), c_int(k),
                               _capi.ptr(out), _capi.ptr(workspace), _capi.stream_ptr(x.device))
    if path is None:
        rc = lib.mxfp4_moe_forward(*args)
    else:
        rc = lib.mxfp4_moe_forward_path(c_int({"fp16": 0, "mxf4": 1}[path]), *args)
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_forward returned {rc}")
    return out


def mma_clocks(n_cols: int = 256, scale_copies: int = 0, iters: int = 2000, device=None) -> float:
    """Tensor-pipe clocks of one `tcgen05.mma kind::mxf4` (M = 128, K = 64, N = n_cols) with `scale_copies` scale-atom
    copies in front of every four MMAs: the library's own microbenchmark (one CTA per SM)."""
    import ctypes
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    scratch = torch.zeros(1, dtype=torch.int64, device=device)
    out = ctypes.c_double(0.0)
    rc = _capi.load("moe").mxfp4_moe_mma_rate(c_int(n_cols), c_int(scale_copies), c_int(iters), _capi.ptr(scratch),
                                              ctypes.cast(ctypes.byref(out), ctypes.c_void_p), _capi.stream_ptr(device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_mma_rate returned {rc}")
    return float(out.value)


STAGES = ("group", "quantise_x", "gemm_gate_up", "quantise_intermediate", "gemm_down", "combine")


def stage_timing(enable: bool) -> bool:
    """Switch the stage timing of the block-scaled batched path on or off (diagnostic: a timed call loses the overlap
    of programmatic dependent launch); returns the previous setting."""
    return bool(_capi.load("moe").mxfp4_moe_stage_timing(c_int(1 if enable else 0)))


def stage_times() -> Dict[str, float]:
    """Microseconds per stage of the last call made while stage timing was on (synchronises on its last event)."""
    import ctypes
    buf = (ctypes.c_float * len(STAGES))()
    rc = _capi.load("moe").mxfp4_moe_stage_times(ctypes.cast(buf, ctypes.c_void_p))
    if rc != 0:
        raise RuntimeError("no timed call of the batched layer to report")
    return {name: float(buf[i]) for i, name in enumerate(STAGES)}


def moe_device_status() -> int:
    """0 unless a kernel of the batched library gave up on a bounded wait or met a bad expert id (synchronises)."""
    return int(_capi.load("moe").mxfp4_moe_device_status())


__all__ = ["moe_forward", "forward_workspace_bytes", "moe_device_status"]
