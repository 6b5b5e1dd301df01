"""B200-native (sm_100a) MXFP4 / FP8 quantized-weight GEMV kernels behind the reference's C ABI.

The directory name carries a hyphen, so it cannot be imported by name; load it with
`__graft_entry__.load_package()` at the repository root, or add the directory's parent to
`sys.path` and import it through `importlib` under the alias `dsv4_b200`.

Layout
------
csrc/      CUDA sources of the three shared libraries (Makefile in this directory builds them into lib/)
lib/       built libraries: libmxfp4_grouped_gemv.so, libmxfp4_gemv.so, libfp8_e4m3_gemv.so, libmxfp4_moe.so
runtime/   host-side mirror of the reference's ctypes bindings (same function names and argument meaning),
           plus the routed-expert bank / router / expert-parallel helpers

There is no CPU fallback: every operator raises if its shared library is missing.
"""
from __future__ import annotations

import os
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(PKG_DIR, "lib")

LIB_FILES = {
    "grouped": "libmxfp4_grouped_gemv.so",
    "mxfp4": "libmxfp4_gemv.so",
    "fp8": "libfp8_e4m3_gemv.so",
    "moe": "libmxfp4_moe.so",
}

# Same override variables as the reference's bindings (runtime/mxfp4_grouped_gemv_binding.py:31-36,
# runtime/mxfp4_gemv_binding.py:18-23, runtime/fp8_e4m3_gemv_binding.py:28-33).
LIB_ENV = {
    "grouped": "MXFP4_GROUPED_LIB",
    "mxfp4": "MXFP4_GEMV_LIB",
    "fp8": "FP8_E4M3_GEMV_LIB",
    "moe": "MXFP4_MOE_LIB",
}


def lib_path(key: str) -> str:
    """Path of one of the three libraries, honouring the reference's environment overrides."""
    return os.path.abspath(os.environ.get(LIB_ENV[key], os.path.join(LIB_DIR, LIB_FILES[key])))


def build(verbose: bool = False) -> None:
    """Compile all CUDA sources for sm_100a with nvcc (no GPU needed)."""
    cmd = ["make", "-C", PKG_DIR, "all"]
    if verbose:
        cmd.append("PTXAS_V=-Xptxas -v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc build failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    for key in LIB_FILES:
        if not os.path.exists(os.path.join(LIB_DIR, LIB_FILES[key])):
            raise RuntimeError(f"build did not produce {LIB_FILES[key]}")
