"""Generates tests/golden/reference_vectors.npz by running the REFERENCE's own Python modules.

Run where the reference tree is mounted (it is not needed at test time):

    python tests/golden/make_golden.py [/path/to/reference]

Every array is an output of unmodified reference code on the inputs stored beside it:
  runtime/mxfp4_unpack.py   mxfp4_unpack, mxfp4_pack
  runtime/e8m0_decode.py    e8m0_decode, e8m0_decode_torch
  runtime/mxfp4_loader.py   MXFP4Loader.dequant_mxfp4 (on a synthetic safetensors snapshot)
  runtime/dsv4_engine_mxfp4.py  DSv4EngineMXFP4._fp8_dequant_to_bf16, DSv4EngineMXFP4._route
Floating-point outputs are stored as raw bit patterns so that NaN and -0.0 survive.
"""
import json
import os
import sys
import tempfile
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DSV4_REFERENCE_ROOT", "/root/reference")
sys.path.insert(0, os.path.join(REF, "runtime"))

import e8m0_decode as ref_e8m0            # noqa: E402
import mxfp4_unpack as ref_fp4            # noqa: E402
import mxfp4_loader as ref_loader         # noqa: E402
import dsv4_engine_mxfp4 as ref_engine    # noqa: E402
from safetensors.torch import save_file   # noqa: E402

out = {}
rng = np.random.default_rng(20240511)

# 1. nibble unpack of every byte value, and the pack inverse
all_bytes = np.arange(256, dtype=np.uint8)
vals = ref_fp4.mxfp4_unpack(all_bytes, (512,), dtype=torch.float32)
out["fp4_all_bytes_in"] = all_bytes
out["fp4_all_bytes_out_bits"] = vals.numpy().view(np.uint32)
out["fp4_pack_roundtrip"] = ref_fp4.mxfp4_pack(vals)

# 2. E8M0 decode of every byte value (numpy and torch variants)
out["e8m0_all_bytes_bits"] = ref_e8m0.e8m0_decode(all_bytes).view(np.uint32)
out["e8m0_all_bytes_torch_bits"] = ref_e8m0.e8m0_decode_torch(torch.from_numpy(all_bytes)).numpy().view(np.uint32)

# 3. loader-level MXFP4 dequantisation on a synthetic snapshot
rows, cols = 48, 256
packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
scale = rng.integers(100, 141, size=(rows, cols // 32), dtype=np.uint8)
scale[0, :4] = [0, 1, 254, 255]           # subnormal scale, smallest normal, largest, NaN sentinel
scale[1, 0] = 127
packed[2, :16] = 0x88                      # a block of -0.0
with tempfile.TemporaryDirectory() as d:
    name = "layers.0.ffn.experts.0.w1"
    save_file({name + ".weight": torch.from_numpy(packed).view(torch.int8),
               name + ".scale": torch.from_numpy(scale).view(torch.float8_e8m0fnu)},
              os.path.join(d, "model-00001-of-00001.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": {name + ".weight": "model-00001-of-00001.safetensors",
                                                   name + ".scale": "model-00001-of-00001.safetensors"}}, f)
    with ref_loader.MXFP4Loader(d) as loader:
        deq = loader.dequant_mxfp4(name)
out["mxfp4_packed"] = packed
out["mxfp4_scale"] = scale
out["mxfp4_dequant_bf16_bits"] = deq.view(torch.int16).numpy()

# 4. FP8 block-128 dequantisation (method body needs no engine state beyond a cache attribute)
n, k = 256, 384
w8 = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
w8[0, :256] = np.arange(256, dtype=np.uint8)      # every E4M3 code, incl. both NaN codes
s8 = rng.integers(110, 131, size=(n // 128, k // 128), dtype=np.uint8)
s8[1, 2] = 0
holder = types.SimpleNamespace()
deq8 = ref_engine.DSv4EngineMXFP4._fp8_dequant_to_bf16(holder, torch.from_numpy(w8), torch.from_numpy(s8))
out["fp8_bytes"] = w8
out["fp8_scale"] = s8
out["fp8_dequant_bf16_bits"] = deq8.view(torch.int16).numpy()
out["e4m3_all_bytes_bits"] = torch.from_numpy(all_bytes).view(torch.float8_e4m3fn).float().numpy().view(np.uint32)

# 5. router: sqrt-softplus scores, top-6, normalised * 1.5, cast to bf16 (identity gate so logits pass through)
logits = rng.standard_normal((6, ref_engine.N_EXPERTS)).astype(np.float32)
logits[4, :] = np.round(logits[4, :] * 2) / 2     # many exact ties
logits[5, :] = -100.0                              # all scores underflow to the same value
logits[5, 17] = 3.0
layer = types.SimpleNamespace(router_gate=torch.eye(ref_engine.N_EXPERTS))
ids, w = ref_engine.DSv4EngineMXFP4._route(types.SimpleNamespace(), torch.from_numpy(logits), layer)
out["route_logits"] = logits
out["route_ids"] = ids.numpy()
out["route_w_bf16_bits"] = w.view(torch.int16).numpy()
out["route_scores_bits"] = torch.sqrt(torch.nn.functional.softplus(torch.from_numpy(logits))).numpy().view(np.uint32)

dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
np.savez_compressed(dst, **out)
print("wrote", dst, {k: v.shape for k, v in out.items()})
