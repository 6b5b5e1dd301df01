"""Checkpoint -> resident expert banks: reads the routed-expert (MXFP4) and shared-expert (FP8) tensors of a
DeepSeek-V4-Flash style safetensors snapshot into the stacked layouts the kernels of this package stream.

Tensor names and dtypes are the reference loader's (runtime/mxfp4_loader.py:35-48):

    layers.{L}.ffn.experts.{E}.w{1|2|3}.weight        I8       [rows, cols/2]   two E2M1 nibbles per byte
    layers.{L}.ffn.experts.{E}.w{1|2|3}.scale         F8_E8M0  [rows, cols/32]
    layers.{L}.ffn.shared_experts.w{1|2|3}.weight     F8_E4M3  [rows, cols]
    layers.{L}.ffn.shared_experts.w{1|2|3}.scale      F8_E8M0  [rows/128, cols/128]

and the file set is `model.safetensors.index.json` (name -> shard) plus the shards, as the reference's
`MXFP4Loader` expects (runtime/mxfp4_loader.py:217-239).  Nothing is repacked: the kernels read the checkpoint's byte
layout as it is, so loading is a copy of raw bytes into one tensor per weight kind, [E_local, rows, bytes per row].
With several GPUs, `rank` / `world` select the contiguous range of experts a rank owns (expert e lives on rank
e // (E / world), the split of expert_parallel.py).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Optional, Tuple

import torch

INDEX_FILE = "model.safetensors.index.json"
_KEYS = (("w1", "w1p", "w1s"), ("w3", "w3p", "w3s"), ("w2", "w2p", "w2s"))


class SnapshotReader:
    """Lazy reader of a sharded safetensors snapshot: every shard is opened at most once."""

    def __init__(self, snapshot_dir: str):
        self.dir = snapshot_dir
        index = os.path.join(snapshot_dir, INDEX_FILE)
        if not os.path.exists(index):
            raise FileNotFoundError(f"{INDEX_FILE} not found in {snapshot_dir}")
        with open(index) as f:
            self.weight_map: Dict[str, str] = json.load(f)["weight_map"]
        self._open = {}

    def _shard(self, name: str):
        from safetensors import safe_open
        if name not in self.weight_map:
            raise KeyError(f"tensor {name!r} is not in the snapshot index")
        shard = self.weight_map[name]
        if shard not in self._open:
            self._open[shard] = safe_open(os.path.join(self.dir, shard), framework="pt", device="cpu")
        return self._open[shard]

    def raw_bytes(self, name: str, dtypes: Iterable[torch.dtype]) -> torch.Tensor:
        """The tensor as uint8 with its own shape; raises if its dtype is not one of `dtypes` (all one byte wide)."""
        t = self._shard(name).get_tensor(name)
        if t.dtype not in tuple(dtypes):
            raise TypeError(f"{name!r} has dtype {t.dtype}, expected one of {tuple(dtypes)}")
        return t.view(torch.uint8)

    def close(self):
        self._open.clear()


def expert_range(n_experts: int, rank: int = 0, world: int = 1) -> Tuple[int, int]:
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    per = n_experts // world
    return rank * per, (rank + 1) * per


def load_expert_bank(snapshot_dir: str, layer: int, n_experts: int, device="cuda", rank: int = 0, world: int = 1,
                     reader: Optional[SnapshotReader] = None) -> Dict[str, torch.Tensor]:
    """The routed experts [lo, hi) of one layer as a bank: w1p / w3p [E_local, hidden, K/2], w2p [E_local, K, hidden/2]
    and the E8M0 scales w1s / w3s / w2s, uint8 on `device` - what mxfp4_grouped_gemv_ids, moe_decode_layer and
    moe_forward take."""
    own = reader is None
    reader = reader or SnapshotReader(snapshot_dir)
    lo, hi = expert_range(n_experts, rank, world)
    bank: Dict[str, torch.Tensor] = {}
    try:
        for e in range(lo, hi):
            for w, pk, sk in _KEYS:
                base = f"layers.{layer}.ffn.experts.{e}.{w}"
                packed = reader.raw_bytes(base + ".weight", (torch.int8, torch.uint8))
                scale = reader.raw_bytes(base + ".scale", (torch.float8_e8m0fnu, torch.uint8))
                rows, half = packed.shape
                if tuple(scale.shape) != (rows, half // 16):
                    raise ValueError(f"{base}: scale shape {tuple(scale.shape)} does not match weight {tuple(packed.shape)} "
                                     f"(one E8M0 byte per 32 elements of a row)")
                if e == lo:
                    bank[pk] = torch.empty((hi - lo, rows, half), dtype=torch.uint8, device=device)
                    bank[sk] = torch.empty((hi - lo, rows, half // 16), dtype=torch.uint8, device=device)
                elif tuple(bank[pk].shape[1:]) != (rows, half):
                    raise ValueError(f"{base}: shape {tuple(packed.shape)} differs from expert {lo}'s")
                bank[pk][e - lo].copy_(packed, non_blocking=False)
                bank[sk][e - lo].copy_(scale, non_blocking=False)
    finally:
        if own:
            reader.close()
    if (bank["w1p"].shape != bank["w3p"].shape or bank["w2p"].shape[1] != bank["w1p"].shape[2] * 2
            or bank["w2p"].shape[2] * 2 != bank["w1p"].shape[1]):
        raise ValueError("w1 / w3 / w2 shapes of the snapshot are not those of one gated FFN")
    return bank


def load_shared_expert_fp8(snapshot_dir: str, layer: int, device="cuda",
                           reader: Optional[SnapshotReader] = None) -> Dict[str, torch.Tensor]:
    """The shared expert of one layer: w1 / w3 [hidden, K], w2 [K, hidden] E4M3 bytes and their E8M0 tile scales
    [rows/128, cols/128], uint8 on `device` - the operands of fp8_e4m3_gemv."""
    own = reader is None
    reader = reader or SnapshotReader(snapshot_dir)
    out: Dict[str, torch.Tensor] = {}
    try:
        for w in ("w1", "w3", "w2"):
            base = f"layers.{layer}.ffn.shared_experts.{w}"
            weight = reader.raw_bytes(base + ".weight", (torch.float8_e4m3fn, torch.uint8))
            scale = reader.raw_bytes(base + ".scale", (torch.float8_e8m0fnu, torch.uint8))
            rows, cols = weight.shape
            if rows % 128 or cols % 128 or tuple(scale.shape) != (rows // 128, cols // 128):
                raise ValueError(f"{base}: weight {tuple(weight.shape)} / scale {tuple(scale.shape)} are not 128x128 tiles")
            out[w] = weight.to(device)
            out[w + "s"] = scale.to(device)
    finally:
        if own:
            reader.close()
    return out


__all__ = ["SnapshotReader", "expert_range", "load_expert_bank", "load_shared_expert_fp8", "INDEX_FILE"]
