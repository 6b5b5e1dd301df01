"""ctypes loading of the three shared libraries, with the exact C signatures of include/dsv4_b200.h."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_longlong, c_size_t, c_void_p, c_float

from .. import lib_path

_P = c_void_p

# symbol -> (restype, argtypes); one table per library
SIGNATURES = {
    "grouped": {
        "mxfp4_grouped_gemv_topk": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P]),
        "mxfp4_grouped_gemv_topk_static": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P]),
        "mxfp4_grouped_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
        "mxfp4_grouped_gemv_topk_ids": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P]),
        "mxfp4_grouped_gemv_topk_ids_stages": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, c_int, _P]),
        "mxfp4_moe_decode_layer": (c_int, [_P] * 8 + [c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_int, _P, _P, _P]),
        "mxfp4_moe_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
        "mxfp4_moe_route_topk": (c_int, [_P, c_int, c_int, c_int, c_int, c_float, c_float, _P, _P, _P]),
        "mxfp4_dequant_bf16": (c_int, [_P, _P, c_longlong, c_int, _P, _P]),
        "dsv4_b200_device_status": (c_int, []),
        "dsv4_b200_set_launch_mode": (c_int, [c_int]),
        "dsv4_b200_test_wait_limits": (c_int, [c_longlong, c_int]),
    },
    "mxfp4": {
        "mxfp4_gemv_m1": (c_int, [_P, _P, _P, c_int, c_int, c_int64, c_int64, _P, _P]),
    },
    "moe": {
        "mxfp4_moe_forward": (c_int, [_P] * 9 + [c_int] * 6 + [_P, _P, _P]),
        "mxfp4_moe_forward_path": (c_int, [c_int] + [_P] * 9 + [c_int] * 6 + [_P, _P, _P]),
        "mxfp4_moe_forward_workspace_bytes": (c_size_t, [c_int] * 6),
        "mxfp4_moe_forward_ep": (c_int, [_P] * 9 + [c_int] * 6 + [_P] + [c_int] * 3 + [_P, _P]),
        "mxfp4_moe_ep_sum": (c_int, [_P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P]),
        "mxfp4_moe_forward_ep2_workspace_bytes": (c_size_t, [c_int] * 7),
        "mxfp4_moe_forward_ep2": (c_int, [_P] * 9 + [c_int] * 6 + [_P] + [c_int] * 2 + [_P, _P]),
        "mxfp4_moe_device_status": (c_int, []),
        "mxfp4_moe_mma_rate": (c_int, [c_int, c_int, c_int, _P, _P, _P]),
        "mxfp4_moe_stage_timing": (c_int, [c_int]),
        "mxfp4_moe_stage_times": (c_int, [_P]),
    },
    "fp8": {
        "fp8_e4m3_gemv_m1": (c_int, [_P, _P, _P, c_int, c_int, c_int64, c_int64, _P, _P]),
        "fp8_e4m3_gemv_m1_f32scale": (c_int, [_P, _P, _P, c_int, c_int, c_int64, c_int64, _P, _P]),
        "fp8_e4m3_gemv_batched": (c_int, [_P, _P, _P, c_int, c_int, c_int64, c_int64, c_int, c_int, c_int64, c_int64,
                                          _P, _P]),
        "fp8_e4m3_shared_swiglu_workspace_bytes": (c_size_t, [c_int]),
        "fp8_e4m3_shared_swiglu_m1": (c_int, [_P] * 7 + [c_int] * 3 + [c_float] * 2 + [_P] * 3),
    },
}

_loaded: dict[str, ctypes.CDLL] = {}


def load(key: str) -> ctypes.CDLL:
    """Load one library (once) and type its entry points.  Raises if the file or a symbol is missing."""
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    path = lib_path(key)
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{os.path.basename(path)} not found at {path}: build it with `make` in the package directory "
            f"(there is no CPU fallback)")
    # RTLD_GLOBAL: the reference's engine resolves these symbols from the global namespace
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    for name, (restype, argtypes) in SIGNATURES[key].items():
        fn = getattr(lib, name)      # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _loaded[key] = lib
    return lib


def ptr(t) -> c_void_p:
    return c_void_p(t.data_ptr())


def stream_ptr(device, stream=None) -> c_void_p:
    import torch
    s = stream if stream is not None else torch.cuda.current_stream(device)
    return c_void_p(s.cuda_stream)
