"""Checkpoint adaptor on CPU: a synthetic snapshot in the reference's naming and dtypes (runtime/mxfp4_loader.py:35-48)
comes back as the stacked banks, byte for byte, whole or as one rank's share."""
import importlib
import json
import os

import pytest
import torch
from safetensors.torch import save_file


@pytest.fixture(scope="module")
def loader(pkg):
    import __graft_entry__ as entry
    return importlib.import_module(entry.PKG_ALIAS + ".runtime.bank_loader")


def _snapshot(tmp, layer, E, K, H, shards=2):
    g = torch.Generator().manual_seed(5)
    tensors, ref = [dict() for _ in range(shards)], {}
    for e in range(E):
        for w, rows, cols in (("w1", H, K), ("w3", H, K), ("w2", K, H)):
            p = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8)
            s = torch.randint(100, 140, (rows, cols // 32), generator=g, dtype=torch.uint8)
            base = f"layers.{layer}.ffn.experts.{e}.{w}"
            tensors[e % shards][base + ".weight"] = p.view(torch.int8)
            tensors[e % shards][base + ".scale"] = s.view(torch.float8_e8m0fnu)
            ref[(e, w)] = (p, s)
    for w, rows, cols in (("w1", 256, 384), ("w3", 256, 384), ("w2", 384, 256)):
        base = f"layers.{layer}.ffn.shared_experts.{w}"
        p = torch.randint(0, 120, (rows, cols), generator=g, dtype=torch.uint8)
        s = torch.randint(110, 130, (rows // 128, cols // 128), generator=g, dtype=torch.uint8)
        tensors[0][base + ".weight"] = p.view(torch.float8_e4m3fn)
        tensors[0][base + ".scale"] = s.view(torch.float8_e8m0fnu)
        ref[("shared", w)] = (p, s)
    weight_map = {}
    for i, t in enumerate(tensors):
        name = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        save_file(t, os.path.join(tmp, name))
        weight_map.update({k: name for k in t})
    with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    return ref


def test_bank_round_trip_and_rank_share(loader, tmp_path):
    E, K, H = 8, 128, 64
    ref = _snapshot(str(tmp_path), 3, E, K, H)
    bank = loader.load_expert_bank(str(tmp_path), 3, E, device="cpu")
    assert bank["w1p"].shape == (E, H, K // 2) and bank["w2p"].shape == (E, K, H // 2)
    assert bank["w1s"].shape == (E, H, K // 32) and bank["w2s"].shape == (E, K, H // 32)
    for e in range(E):
        for w, pk, sk in (("w1", "w1p", "w1s"), ("w3", "w3p", "w3s"), ("w2", "w2p", "w2s")):
            assert torch.equal(bank[pk][e], ref[(e, w)][0]) and torch.equal(bank[sk][e], ref[(e, w)][1])
    share = loader.load_expert_bank(str(tmp_path), 3, E, device="cpu", rank=1, world=4)
    assert share["w1p"].shape[0] == 2
    assert torch.equal(share["w3p"], bank["w3p"][2:4]) and torch.equal(share["w2s"], bank["w2s"][2:4])
    shared = loader.load_shared_expert_fp8(str(tmp_path), 3, device="cpu")
    for w in ("w1", "w3", "w2"):
        assert torch.equal(shared[w], ref[("shared", w)][0]) and torch.equal(shared[w + "s"], ref[("shared", w)][1])


def test_errors(loader, tmp_path):
    _snapshot(str(tmp_path), 0, 4, 64, 32, shards=1)
    with pytest.raises(KeyError):
        loader.load_expert_bank(str(tmp_path), 1, 4, device="cpu")          # no such layer
    with pytest.raises(ValueError):
        loader.load_expert_bank(str(tmp_path), 0, 4, device="cpu", world=3)  # experts do not split
    with pytest.raises(FileNotFoundError):
        loader.SnapshotReader(str(tmp_path / "nowhere"))
