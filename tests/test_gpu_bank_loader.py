"""Checkpoint adaptor on the GPU: a synthetic snapshot written in the reference's naming and dtypes
(runtime/mxfp4_loader.py:35-48, 217-239: `I8` packed weights, `F8_E8M0` scales, `F8_E4M3` shared-expert weights) is
loaded onto the device by `load_expert_bank` / `load_shared_expert_fp8` - whole and as one rank's share - and fed to
the kernels; the outputs are checked against the CPU oracle on the tensors that were written."""
import importlib
import json
import os

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import oracle

pytestmark = pytest.mark.gpu


def write_snapshot(tmp, layer, bank, shared, shards=2):
    E = bank["w1p"].shape[0]
    tensors = [dict() for _ in range(shards)]
    for e in range(E):
        for w in ("w1", "w3", "w2"):
            base = f"layers.{layer}.ffn.experts.{e}.{w}"
            tensors[e % shards][base + ".weight"] = bank[w + "p"][e].contiguous().view(torch.int8)
            tensors[e % shards][base + ".scale"] = bank[w + "s"][e].contiguous().view(torch.float8_e8m0fnu)
    for w in ("w1", "w3", "w2"):
        base = f"layers.{layer}.ffn.shared_experts.{w}"
        tensors[0][base + ".weight"] = shared[w].contiguous().view(torch.float8_e4m3fn)
        tensors[0][base + ".scale"] = shared[w + "s"].contiguous().view(torch.float8_e8m0fnu)
    weight_map = {}
    for i, t in enumerate(tensors):
        name = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        save_file(t, os.path.join(tmp, name))
        weight_map.update({k: name for k in t})
    with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)


def test_loaded_bank_feeds_the_kernels(rt, qz, pkg, tmp_path):
    loader = importlib.import_module("dsv4_b200.runtime.bank_loader")
    dev = torch.device("cuda:0")
    E, K, H, k, layer = 8, 1024, 1024, 6, 5
    bank = qz.make_expert_bank(E, K, H, "cpu", seed=55)
    g = torch.Generator().manual_seed(56)
    shared = {}
    for w, rows, cols in (("w1", H, K), ("w3", H, K), ("w2", K, H)):
        shared[w], shared[w + "s"] = qz.quantize_fp8_block128(torch.randn(rows, cols, generator=g) * 0.02, "e8m0")
    write_snapshot(str(tmp_path), layer, bank, shared)

    x = torch.randn(K, generator=g).to(torch.bfloat16)
    logits = torch.randn(E, generator=g)
    ids, w = oracle.route_softmax(logits.numpy()[None], k)
    ref = oracle.moe_layer_ref(x[None], bank, ids, w)[0]

    # the whole bank on one device: one decode layer (router + FFN in one call)
    dbank = loader.load_expert_bank(str(tmp_path), layer, E, device=dev)
    assert all(t.is_cuda for t in dbank.values())
    out = rt.moe_decode_layer(dbank, logits.to(dev), x.to(dev), k=k, score_func="softmax")
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    assert oracle.max_abs_rel(got, ref) <= 1e-2 and oracle.cosine(got, ref) >= 0.9999

    # one rank's share (rank 1 of 2 holds experts 4..7): the picks that live there, through the index entry
    share = loader.load_expert_bank(str(tmp_path), layer, E, device=dev, rank=1, world=2)
    lo, hi = loader.expert_range(E, 1, 2)
    local = [(int(e) - lo, float(wt)) for e, wt in zip(ids[0], w[0]) if lo <= e < hi]
    assert local, "seed leaves rank 1 without a pick"
    lids = torch.tensor([e for e, _ in local], dtype=torch.int32, device=dev)
    lw = torch.tensor([wt for _, wt in local], dtype=torch.float32, device=dev)
    part = rt.mxfp4_grouped_gemv_ids(share, lids, x.to(dev), lw)
    torch.cuda.synchronize()
    keep = np.array([[wt if lo <= e < hi else 0.0 for e, wt in zip(ids[0], w[0])]], dtype=np.float32)
    ref_part = oracle.moe_layer_ref(x[None], bank, ids, keep)[0]
    gp = part.float().cpu().numpy()
    assert oracle.max_abs_rel(gp, ref_part) <= 1e-2 and oracle.cosine(gp, ref_part) >= 0.9999

    # the shared expert's FP8 tensors through the fused shared-expert entry
    dsh = loader.load_shared_expert_fp8(str(tmp_path), layer, device=dev)
    y = rt.fp8_shared_swiglu(dsh, x.to(dev))
    torch.cuda.synchronize()
    ref_sh = oracle.shared_swiglu_fp8_ref(x, shared)
    gs = y.float().cpu().numpy()
    assert oracle.max_abs_rel(gs, ref_sh) <= 1e-2 and oracle.cosine(gs, ref_sh) >= 0.9999
    assert rt.device_status() == 0
