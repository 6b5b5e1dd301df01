"""CPU oracle for the quantized-weight GEMV/GEMM path.

TEST INFRASTRUCTURE ONLY.  This package is a CPU restatement (numpy, with torch
only for bf16 rounding and the FP32 matmul) of the reference's own Python
dequantisation path and of the arithmetic its CUDA kernels perform.  Nothing
on the product path may import it: only the test-suite, the smoke check and
the benchmark's CPU-baseline / reference legs do, and only as the checker or
as the timed CPU baseline.

Pinning status
--------------
* dequantisation (nibble unpack, E8M0 decode, MXFP4 -> bf16, FP8-E4M3 block
  dequant), the router score / top-K rule and the pack/unpack inverse are
  PINNED: they are checked bit-for-bit against vectors produced by importing the
  reference's modules (tests/golden/make_golden.py, committed with its output).
* the GEMV / MoE outputs have no golden vector in the reference (it ships no
  test-suite); they are pinned one level down: pinned dequant followed by an
  FP32 matmul, which is exactly how the reference defines its ground truth
  (runtime/mxfp4_loader.py:272-309 "ground-truth comparisons").
* the BF16 -> MXFP4 / FP8 quantiser used to make synthetic weights is
  PARITY UNPINNED: the reference contains no quantiser (weights arrive
  pre-quantised).  It cannot influence kernel-vs-oracle parity, because both
  sides consume the same bytes.
"""
from .mxfp4_ref import *  # noqa: F401,F403
