"""Routed-expert MXFP4 grouped GEMV operator — same call as the reference's
runtime/mxfp4_grouped_gemv_binding.py:95-174:

    out = mxfp4_grouped_gemv(W1, W3, W2, scales, x, r)

W1 / W3 / W2 are dicts {'packed': uint8, 'scale': uint8} stacked over the n_exp selected experts
(W1, W3 packed [n_exp, hidden, K_in/2], scale [n_exp, hidden, K_in/32]; W2 packed [n_exp, out_dim, hidden/2],
scale [n_exp, out_dim, hidden/32]); `scales` is ignored as in the reference; x bfloat16 [K_in]; r float32 [n_exp].
Returns bfloat16 [out_dim].  ValueError on a bad argument, RuntimeError on a non-zero return code.

Additions with no counterpart in the reference: `mxfp4_grouped_gemv_ids` (experts taken from a resident bank by
index: no gather copy), `moe_route_topk` (router scores / top-k / weights on the device) and `mxfp4_dequant_bf16`.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Any, Dict, Optional

import torch

from . import _capi

MXFP4_BLOCK_ELEMS = 32


def _check(t: torch.Tensor, name: str, dtype: torch.dtype) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name}: expected CUDA tensor, got device={t.device}")
    if t.dtype != dtype:
        raise ValueError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: tensor must be contiguous")


def _check_expert_set(W1, W3, W2, K_in):
    for name, w in (("W1", W1), ("W3", W3), ("W2", W2)):
        if "packed" not in w or "scale" not in w:
            raise ValueError(f"{name} must contain 'packed' and 'scale' tensors")
        _check(w["packed"], f"{name}.packed", torch.uint8)
        _check(w["scale"], f"{name}.scale", torch.uint8)
    n, hidden = W1["packed"].shape[0], W1["packed"].shape[1]
    out_dim = W2["packed"].shape[1]
    b = MXFP4_BLOCK_ELEMS
    expect = {
        "W1.packed": (W1["packed"], (n, hidden, K_in // 2)), "W3.packed": (W3["packed"], (n, hidden, K_in // 2)),
        "W1.scale": (W1["scale"], (n, hidden, K_in // b)), "W3.scale": (W3["scale"], (n, hidden, K_in // b)),
        "W2.packed": (W2["packed"], (n, out_dim, hidden // 2)), "W2.scale": (W2["scale"], (n, out_dim, hidden // b)),
    }
    for name, (t, shape) in expect.items():
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} shape {tuple(t.shape)} != {shape}")
    return n, hidden, out_dim


def workspace_bytes(n_exp: int, hidden: int, out_dim: int) -> int:
    return int(_capi.load("grouped").mxfp4_grouped_workspace_bytes(n_exp, hidden, out_dim))


def mxfp4_grouped_gemv(W1: Dict[str, torch.Tensor], W3: Dict[str, torch.Tensor], W2: Dict[str, torch.Tensor],
                       scales: Any, x: torch.Tensor, r: torch.Tensor, out: Optional[torch.Tensor] = None,
                       workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    del scales
    lib = _capi.load("grouped")
    _check(x, "x", torch.bfloat16)
    _check(r, "r", torch.float32)
    K_in = x.numel()
    n_exp, hidden, out_dim = _check_expert_set(W1, W3, W2, K_in)
    if tuple(r.shape) != (n_exp,):
        raise ValueError(f"r shape {tuple(r.shape)} != ({n_exp},)")
    if out is None:
        out = torch.empty(out_dim, dtype=torch.bfloat16, device=x.device)
    if workspace is None:
        workspace = torch.empty(workspace_bytes(n_exp, hidden, out_dim), dtype=torch.uint8, device=x.device)
    rc = lib.mxfp4_grouped_gemv_topk(
        _capi.ptr(x), _capi.ptr(W1["packed"]), _capi.ptr(W3["packed"]), _capi.ptr(W2["packed"]),
        _capi.ptr(W1["scale"]), _capi.ptr(W3["scale"]), _capi.ptr(W2["scale"]), _capi.ptr(r),
        c_int(K_in), c_int(hidden), c_int(out_dim), c_int(n_exp), _capi.ptr(out), _capi.ptr(workspace),
        _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_grouped_gemv_topk returned {rc}")
    return out


def mxfp4_grouped_gemv_static(W1: Dict[str, torch.Tensor], W3: Dict[str, torch.Tensor], W2: Dict[str, torch.Tensor],
                              x: torch.Tensor, r: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The routed-expert FFN through the entry point that takes no workspace and allocates nothing.

    For hosts that cannot get device memory at call time (everything already committed to the expert bank and the
    KV cache, or a thread that must not enter cudaMalloc): the intermediate sits in a fixed 96 KB array inside the
    library, shared by every call on the device, so calls that overlap on the GPU must be serialised by the caller.
    `out` (bfloat16 [out_dim]) is mandatory so that this wrapper allocates nothing either.  hidden <= 4096,
    six experts.  Make the first call on a device before capturing a stream there."""
    lib = _capi.load("grouped")
    _check(x, "x", torch.bfloat16)
    _check(r, "r", torch.float32)
    K_in = x.numel()
    n_exp, hidden, out_dim = _check_expert_set(W1, W3, W2, K_in)
    if tuple(r.shape) != (n_exp,):
        raise ValueError(f"r shape {tuple(r.shape)} != ({n_exp},)")
    _check(out, "out", torch.bfloat16)
    if tuple(out.shape) != (out_dim,):
        raise ValueError(f"out shape {tuple(out.shape)} != ({out_dim},)")
    rc = lib.mxfp4_grouped_gemv_topk_static(
        _capi.ptr(x), _capi.ptr(W1["packed"]), _capi.ptr(W3["packed"]), _capi.ptr(W2["packed"]),
        _capi.ptr(W1["scale"]), _capi.ptr(W3["scale"]), _capi.ptr(W2["scale"]), _capi.ptr(r),
        c_int(K_in), c_int(hidden), c_int(out_dim), c_int(n_exp), _capi.ptr(out), _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_grouped_gemv_topk_static returned {rc}")
    return out


def mxfp4_grouped_gemv_ids(bank: Dict[str, torch.Tensor], ids: torch.Tensor, x: torch.Tensor, r: torch.Tensor,
                           out: Optional[torch.Tensor] = None,
                           workspace: Optional[torch.Tensor] = None, stage_mask: int = 3,
                           check: bool = True) -> torch.Tensor:
    """Same FFN, experts `ids` (int32 CUDA [n_exp]) picked from a resident bank
    {'w1p','w3p','w2p','w1s','w3s','w2s'} stacked over ALL experts.  `stage_mask` 1 / 2 runs only the gate-up /
    the down kernel (profiling); `check=False` skips the Python-side shape checks for callers that made them once."""
    lib = _capi.load("grouped")
    K_in = x.numel()
    n_exp = ids.numel()
    if check:
        _check(x, "x", torch.bfloat16)
        _check(r, "r", torch.float32)
        _check(ids, "ids", torch.int32)
        _, hidden, out_dim = _check_expert_set({"packed": bank["w1p"], "scale": bank["w1s"]},
                                               {"packed": bank["w3p"], "scale": bank["w3s"]},
                                               {"packed": bank["w2p"], "scale": bank["w2s"]}, K_in)
        if tuple(r.shape) != (n_exp,):
            raise ValueError(f"r shape {tuple(r.shape)} != ({n_exp},)")
    else:
        hidden, out_dim = bank["w1p"].shape[1], bank["w2p"].shape[1]
    if out is None:
        out = torch.empty(out_dim, dtype=torch.bfloat16, device=x.device)
    if workspace is None:
        workspace = torch.empty(workspace_bytes(n_exp, hidden, out_dim), dtype=torch.uint8, device=x.device)
    rc = lib.mxfp4_grouped_gemv_topk_ids_stages(
        _capi.ptr(x), _capi.ptr(bank["w1p"]), _capi.ptr(bank["w3p"]), _capi.ptr(bank["w2p"]),
        _capi.ptr(bank["w1s"]), _capi.ptr(bank["w3s"]), _capi.ptr(bank["w2s"]), _capi.ptr(ids), _capi.ptr(r),
        c_int(K_in), c_int(hidden), c_int(out_dim), c_int(n_exp), _capi.ptr(out), _capi.ptr(workspace),
        c_int(stage_mask), _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_grouped_gemv_topk_ids returned {rc}")
    return out


def moe_route_topk(logits: torch.Tensor, k: int = 6, score_func: str = "sqrt_softplus", eps: float = 1e-20,
                   scaling: float = 1.5, ids_out: Optional[torch.Tensor] = None,
                   w_out: Optional[torch.Tensor] = None):
    """Router on the device: logits float32 [T, E] -> (ids int32 [T, k], weights float32 [T, k]).

    score_func 'sqrt_softplus' is the engine's rule (kernel/cpp-engine-mxfp4/routed.cu:156-208, Python twin
    runtime/dsv4_engine_mxfp4.py:363-370); 'softmax' renormalises softmax probabilities over the k picks.
    """
    lib = _capi.load("grouped")
    _check(logits, "logits", torch.float32)
    if logits.dim() == 1:
        logits = logits.unsqueeze(0)
    T, E = logits.shape
    func = {"softmax": 0, "sqrt_softplus": 1}[score_func]
    ids = ids_out if ids_out is not None else torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = w_out if w_out is not None else torch.empty(T, k, dtype=torch.float32, device=logits.device)
    rc = lib.mxfp4_moe_route_topk(_capi.ptr(logits), c_int(T), c_int(E), c_int(k), c_int(func), c_float(eps),
                                  c_float(scaling), _capi.ptr(ids), _capi.ptr(w), _capi.stream_ptr(logits.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_route_topk returned {rc}")
    return ids, w


def moe_decode_layer(bank: Dict[str, torch.Tensor], logits: torch.Tensor, x: torch.Tensor, k: int = 6,
                     score_func: str = "sqrt_softplus", eps: float = 1e-20, scaling: float = 1.5,
                     out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                     check: bool = True) -> torch.Tensor:
    """One decode layer for one token: router + routed-expert FFN over a resident bank, in one call.

    logits float32 [n_experts], x bfloat16 [K_in]; returns bfloat16 [out_dim].  Pass `workspace` (uint8,
    `decode_workspace_bytes`) to read the picks afterwards with `decode_picks`."""
    lib = _capi.load("grouped")
    K_in, n_experts = x.numel(), logits.numel()
    hidden, out_dim = bank["w1p"].shape[1], bank["w2p"].shape[1]
    if check:
        _check(x, "x", torch.bfloat16)
        _check(logits, "logits", torch.float32)
        _check_expert_set({"packed": bank["w1p"], "scale": bank["w1s"]}, {"packed": bank["w3p"], "scale": bank["w3s"]},
                          {"packed": bank["w2p"], "scale": bank["w2s"]}, K_in)
        if bank["w1p"].shape[0] != n_experts:
            raise ValueError(f"bank holds {bank['w1p'].shape[0]} experts, logits {n_experts}")
    if out is None:
        out = torch.empty(out_dim, dtype=torch.bfloat16, device=x.device)
    if workspace is None:
        workspace = torch.empty(decode_workspace_bytes(k, hidden, out_dim), dtype=torch.uint8, device=x.device)
    func = {"softmax": 0, "sqrt_softplus": 1}[score_func]
    rc = lib.mxfp4_moe_decode_layer(
        _capi.ptr(x), _capi.ptr(bank["w1p"]), _capi.ptr(bank["w3p"]), _capi.ptr(bank["w2p"]), _capi.ptr(bank["w1s"]),
        _capi.ptr(bank["w3s"]), _capi.ptr(bank["w2s"]), _capi.ptr(logits), c_int(n_experts), c_int(func),
        c_float(eps), c_float(scaling), c_int(K_in), c_int(hidden), c_int(out_dim), c_int(k), _capi.ptr(out),
        _capi.ptr(workspace), _capi.stream_ptr(x.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_moe_decode_layer returned {rc}")
    return out


def decode_workspace_bytes(k: int, hidden: int, out_dim: int) -> int:
    return int(_capi.load("grouped").mxfp4_moe_decode_workspace_bytes(k, hidden, out_dim))


def decode_picks(workspace: torch.Tensor, k: int, hidden: int):
    """(ids int32 [k], weights float32 [k]) left in the workspace by moe_decode_layer."""
    off = k * hidden * 8
    return workspace[off:off + 4 * k].view(torch.int32), workspace[off + 32:off + 32 + 4 * k].view(torch.float32)


def mxfp4_dequant_bf16(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """MXFP4 -> bfloat16 [rows, cols] on the device, scale byte 0xFF -> NaN
    (the semantics of runtime/mxfp4_loader.py:272-309)."""
    lib = _capi.load("grouped")
    _check(packed, "packed", torch.uint8)
    _check(scale, "scale", torch.uint8)
    rows, cols = packed.shape[0], packed.shape[1] * 2
    if tuple(scale.shape) != (rows, cols // 32):
        raise ValueError(f"scale shape {tuple(scale.shape)} != ({rows}, {cols // 32})")
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=packed.device)
    rc = lib.mxfp4_dequant_bf16(_capi.ptr(packed), _capi.ptr(scale), c_longlong(rows), c_int(cols), _capi.ptr(out),
                                _capi.stream_ptr(packed.device))
    if rc != 0:
        raise RuntimeError(f"mxfp4_dequant_bf16 returned {rc}")
    return out


def device_status() -> int:
    """0 unless a kernel gave up on one of its bounded waits since the last call (synchronises the device)."""
    return int(_capi.load("grouped").dsv4_b200_device_status())


LAUNCH_MODES = {"chain": 0, "coop": 1, "auto": 2, "pdl": 3}


def set_launch_mode(mode: str) -> str:
    """How the single-kernel decode path is launched from now on: "auto" (default: the first stream that calls on a
    device with programmatic stream serialisation, every other stream cooperatively - safe from any number of
    streams), "pdl" (programmatic for every stream: only for callers with one stream per device), "coop"
    (cooperative for every stream) or "chain" (two kernels).  Returns the previous mode."""
    before = int(_capi.load("grouped").dsv4_b200_set_launch_mode(c_int(LAUNCH_MODES[mode])))
    return {v: k for k, v in LAUNCH_MODES.items()}.get(before, str(before))


def debug_wait_limits(polls: int, phantom_ctas: int) -> None:
    """Test hook: poll budget of the device-side waits and a number of producers that never arrive; (0, 0) restores
    the defaults."""
    if _capi.load("grouped").dsv4_b200_test_wait_limits(c_longlong(polls), c_int(phantom_ctas)) != 0:
        raise ValueError("bad wait limits")


__all__ = ["device_status", "set_launch_mode", "debug_wait_limits", "moe_decode_layer", "decode_workspace_bytes", "decode_picks", "mxfp4_grouped_gemv", "mxfp4_grouped_gemv_static", "mxfp4_grouped_gemv_ids", "moe_route_topk", "mxfp4_dequant_bf16",
           "workspace_bytes", "MXFP4_BLOCK_ELEMS"]
