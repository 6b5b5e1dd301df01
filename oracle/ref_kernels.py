"""ctypes access to the REFERENCE's CUDA kernels built by oracle/Makefile into oracle/_ref/ (TEST INFRASTRUCTURE).

Used by the GPU tests as a second checker (the reference's own device code on the same inputs) and by the
benchmark as "the reference kernel on this GPU".  `available()` is False when the files were not built.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_size_t, c_void_p

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_P = c_void_p
_libs = {}


def available() -> bool:
    return all(os.path.exists(os.path.join(_DIR, f)) for f in
               ("libmxfp4_grouped_gemv.so", "libmxfp4_gemv.so", "libfp8_e4m3_gemv.so"))


def _lib(name):
    if name not in _libs:
        # RTLD_LOCAL: the reference exports the same symbol names as the product
        _libs[name] = ctypes.CDLL(os.path.join(_DIR, name), mode=ctypes.RTLD_LOCAL)
    return _libs[name]


def grouped_gemv(x, w1p, w3p, w2p, w1s, w3s, w2s, r):
    """kernel/mxfp4-routed/mxfp4_grouped_gemv.cu:294 through its own C ABI; tensors are CUDA, stacked [6, ...]."""
    import torch
    lib = _lib("libmxfp4_grouped_gemv.so")
    lib.mxfp4_grouped_gemv_topk.restype = c_int
    lib.mxfp4_grouped_gemv_topk.argtypes = [_P] * 8 + [c_int] * 4 + [_P] * 3
    lib.mxfp4_grouped_workspace_bytes.restype = c_size_t
    lib.mxfp4_grouped_workspace_bytes.argtypes = [c_int] * 3
    n, hidden, out_dim, k_in = w1p.shape[0], w1p.shape[1], w2p.shape[1], x.numel()
    out = torch.empty(out_dim, dtype=torch.bfloat16, device=x.device)
    ws = torch.empty(lib.mxfp4_grouped_workspace_bytes(n, hidden, out_dim), dtype=torch.uint8, device=x.device)
    rc = lib.mxfp4_grouped_gemv_topk(*[_P(t.data_ptr()) for t in (x, w1p, w3p, w2p, w1s, w3s, w2s, r)],
                                     k_in, hidden, out_dim, n, _P(out.data_ptr()), _P(ws.data_ptr()),
                                     _P(torch.cuda.current_stream(x.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"reference mxfp4_grouped_gemv_topk returned {rc}")
    return out


def _dense(libname, symbol, x, w, s):
    import torch
    lib = _lib(libname)
    fn = getattr(lib, symbol)
    fn.restype = c_int
    fn.argtypes = [_P, _P, _P, c_int, c_int, c_int64, c_int64, _P, _P]
    out = torch.empty(w.shape[0], dtype=torch.bfloat16, device=x.device)
    rc = fn(_P(x.data_ptr()), _P(w.data_ptr()), _P(s.data_ptr()), x.numel(), w.shape[0], w.stride(0), s.stride(0),
            _P(out.data_ptr()), _P(torch.cuda.current_stream(x.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"reference {symbol} returned {rc}")
    return out


def mxfp4_gemv(x, w_packed, w_scale):
    """kernel/mxfp4-dense/mxfp4_gemv.cu:131 through its own C ABI."""
    return _dense("libmxfp4_gemv.so", "mxfp4_gemv_m1", x, w_packed, w_scale)


def fp8_gemv(x, w_fp8, w_scale):
    """kernel/fp8-dense/fp8_e4m3_gemv.cu:132 through its own C ABI."""
    return _dense("libfp8_e4m3_gemv.so", "fp8_e4m3_gemv_m1", x, w_fp8, w_scale)
