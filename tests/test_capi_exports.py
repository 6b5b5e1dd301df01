"""The three shared libraries load and export every symbol include/dsv4_b200.h declares (no GPU needed),
and reject bad arguments with the reference's return codes before touching the device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dsv4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|size_t)\s+(\w+)\s*\(", text)))


def test_header_declares_the_reference_entry_points():
    syms = declared_symbols()
    for name in ("mxfp4_grouped_gemv_topk", "mxfp4_grouped_workspace_bytes", "mxfp4_gemv_m1", "fp8_e4m3_gemv_m1"):
        assert name in syms


def test_every_declared_symbol_is_exported(pkg):
    libs = [ctypes.CDLL(pkg.lib_path(k), mode=ctypes.RTLD_GLOBAL) for k in pkg.LIB_FILES]
    for name in declared_symbols():
        assert any(hasattr(lib, name) for lib in libs), f"{name} is declared but not exported"


def test_library_file_names_match_the_reference(pkg):
    assert os.path.basename(pkg.lib_path("grouped")) == "libmxfp4_grouped_gemv.so"
    assert os.path.basename(pkg.lib_path("mxfp4")) == "libmxfp4_gemv.so"
    assert os.path.basename(pkg.lib_path("fp8")) == "libfp8_e4m3_gemv.so"


def test_env_override_is_honoured(pkg, monkeypatch):
    monkeypatch.setenv("MXFP4_GEMV_LIB", "/nonexistent/libmxfp4_gemv.so")
    assert pkg.lib_path("mxfp4") == "/nonexistent/libmxfp4_gemv.so"


def test_missing_library_fails_loudly(pkg, monkeypatch):
    import importlib
    capi = importlib.import_module("dsv4_b200.runtime._capi")
    monkeypatch.setenv("FP8_E4M3_GEMV_LIB", "/nonexistent/libfp8_e4m3_gemv.so")
    monkeypatch.setattr(capi, "_loaded", {})
    with pytest.raises(FileNotFoundError):
        capi.load("fp8")


def test_workspace_bytes(pkg):
    import importlib
    capi = importlib.import_module("dsv4_b200.runtime._capi")
    lib = capi.load("grouped")
    # the intermediate [n_exp, hidden] as 8-byte {value, tag} words, then the generation word
    assert lib.mxfp4_grouped_workspace_bytes(6, 2048, 4096) == 6 * 2048 * 8 + 64
    assert lib.mxfp4_moe_decode_workspace_bytes(6, 2048, 4096) == 6 * 2048 * 8 + 64 + 64
    assert lib.mxfp4_grouped_workspace_bytes(0, 2048, 4096) == 0


def test_argument_checks_return_the_reference_codes(pkg):
    """These paths return before any CUDA call, so they run without a GPU."""
    import importlib
    capi = importlib.import_module("dsv4_b200.runtime._capi")
    g, d, f = capi.load("grouped"), capi.load("mxfp4"), capi.load("fp8")
    one = ctypes.c_void_p(16)      # never dereferenced on these paths
    args = [one] * 8
    assert g.mxfp4_grouped_gemv_topk(*args, 4095, 2048, 4096, 6, one, one, None) == -1
    assert g.mxfp4_grouped_gemv_topk(*args, 4096, 2040, 4096, 6, one, one, None) == -2
    assert g.mxfp4_grouped_gemv_topk(*args, 8192, 2048, 4096, 6, one, one, None) == -3
    assert g.mxfp4_grouped_gemv_topk(*args, 4096, 2048, 4096, 5, one, one, None) == -4
    assert g.mxfp4_grouped_gemv_topk(*([None] * 8), 4096, 2048, 4096, 6, one, one, None) == -8
    assert g.mxfp4_grouped_gemv_topk_ids(*args, one, 4096, 2048, 4096, 9, one, one, None) == -4
    assert d.mxfp4_gemv_m1(one, one, one, 48, 8, 24, 1, one, None) == -1
    assert d.mxfp4_gemv_m1(one, one, one, 16384, 8, 8192, 512, one, None) == -2
    assert d.mxfp4_gemv_m1(None, one, one, 64, 8, 32, 2, one, None) == -8
    assert d.mxfp4_gemv_m1(None, None, None, 64, 0, 32, 2, None, None) == 0
    assert f.fp8_e4m3_gemv_m1(one, one, one, 192, 128, 192, 1, one, None) == -1
    assert f.fp8_e4m3_gemv_m1(one, one, one, 256, 100, 256, 2, one, None) == -2
    assert f.fp8_e4m3_gemv_m1(one, one, one, 32768, 128, 32768, 256, one, None) == -3
    assert g.mxfp4_moe_route_topk(one, 4, 2048, 6, 1, 0.0, 1.0, one, one, None) == -1
    assert g.mxfp4_moe_route_topk(one, 4, 256, 6, 7, 0.0, 1.0, one, one, None) == -1


def test_bindings_reject_cpu_tensors(rt):
    import torch
    x = torch.zeros(64, dtype=torch.bfloat16)
    wp = torch.zeros(8, 32, dtype=torch.uint8)
    ws = torch.zeros(8, 2, dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        rt.mxfp4_gemv(wp, ws, x)
    with pytest.raises(RuntimeError):
        rt.fp8_e4m3_gemv(torch.zeros(128, 128, dtype=torch.uint8), torch.zeros(1, 1, dtype=torch.uint8),
                         torch.zeros(128, dtype=torch.bfloat16))
    w = {"packed": torch.zeros(6, 32, 32, dtype=torch.uint8), "scale": torch.zeros(6, 32, 2, dtype=torch.uint8)}
    with pytest.raises(ValueError):
        rt.mxfp4_grouped_gemv(w, w, w, None, x, torch.zeros(6))
