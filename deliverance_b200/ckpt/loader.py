"""Checkpoint directory access: single-file or indexed multi-file safetensors, JQ4 pairing and tensor-parallel shards.

Behaviour follows the reference loader (safetensors/src/main/java/io/teknek/deliverance/safetensors/DefaultWeightLoader.java:108-149,
Weights.java:36-56,133-136,249-286, TensorShardSpec): a ``Q4`` entry is paired with its ``.qb`` sidecar, ``.qb``
entries are skipped when the model's majority dtype is inferred, a *row* shard slices output features (dim 0) and a
*column* shard slices input features (last dim) and must be 32-aligned for ``Q4`` weights.
"""
from __future__ import annotations

import json
import os
from collections import Counter
from dataclasses import dataclass
from typing import Optional

import torch

from .jq4 import BLOCK
from .safetensors_io import INDEX_FILE, SINGLE_FILE, Q4Tensor, SafeTensorFile, TensorInfo


@dataclass(frozen=True)
class ShardSpec:
    """Contiguous 1/size slice of one axis. ``axis`` is ``"row"`` (dim 0, output features) or ``"col"`` (last dim)."""

    axis: str
    rank: int
    size: int
    # optional: the axis is made of `groups` equal segments that are each split (fused gate|up, stacked q|k|v)
    groups: int = 1

    def ranges(self, extent: int) -> list[tuple[int, int]]:
        if extent % (self.size * self.groups) != 0:
            raise ValueError(f"extent {extent} is not divisible by {self.size}x{self.groups}")
        seg = extent // self.groups
        per = seg // self.size
        return [(g * seg + self.rank * per, g * seg + (self.rank + 1) * per) for g in range(self.groups)]


class WeightLoader:
    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files: dict[str, SafeTensorFile] = {}
        self._where: dict[str, str] = {}
        index = os.path.join(model_dir, INDEX_FILE)
        single = os.path.join(model_dir, SINGLE_FILE)
        if os.path.exists(index):
            with open(index) as f:
                idx = json.load(f)
            self.index_metadata = idx.get("metadata", {})
            for name, fname in idx["weight_map"].items():
                self._where[name] = fname
            for fname in sorted(set(self._where.values())):
                self._files[fname] = SafeTensorFile(os.path.join(model_dir, fname))
        elif os.path.exists(single):
            self.index_metadata = {}
            self._files[SINGLE_FILE] = SafeTensorFile(single)
            for name in self._files[SINGLE_FILE].names():
                self._where[name] = SINGLE_FILE
        else:
            found = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
            if not found:
                raise FileNotFoundError(f"no safetensors files in {model_dir}")
            self.index_metadata = {}
            for fname in found:
                self._files[fname] = SafeTensorFile(os.path.join(model_dir, fname))
                for name in self._files[fname].names():
                    self._where[name] = fname
        # names present in a file but missing in the index still resolve
        for fname, fh in self._files.items():
            for name in fh.names():
                self._where.setdefault(name, fname)

    # -- inventory -------------------------------------------------------------------------------------------------
    def names(self) -> list[str]:
        return [n for n in self._where if not n.endswith(".qb")]

    def has(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str) -> TensorInfo:
        return self._files[self._where[name]].infos[name]

    def is_q4(self, name: str) -> bool:
        return self.has(name) and self.info(name).dtype == "Q4"

    def majority_dtype(self) -> str:
        """Most common dtype by tensor count, ignoring ``.qb`` sidecars."""
        c = Counter(self.info(n).dtype for n in self.names())
        return c.most_common(1)[0][0] if c else "F32"

    def metadata(self) -> dict:
        out: dict = {}
        for fh in self._files.values():
            out.update(fh.metadata)
        return out

    # -- loading ---------------------------------------------------------------------------------------------------
    def load(self, name: str, shard: Optional[ShardSpec] = None):
        """Return a dense ``torch.Tensor`` view or a :class:`Q4Tensor`; ``shard`` selects this rank's slice."""
        if not self.has(name):
            raise KeyError(f"tensor '{name}' not found in {self.model_dir}")
        fh = self._files[self._where[name]]
        info = fh.infos[name]
        if info.dtype == "Q4":
            qb = name + ".qb"
            if not self.has(qb):
                raise KeyError(f"Q4 tensor '{name}' has no '.qb' scale sidecar")
            packed = fh.tensor(name)
            scales = self._files[self._where[qb]].tensor(qb).reshape(*info.shape[:-1], info.shape[-1] // BLOCK)
            q = Q4Tensor(packed, scales, info.shape)
            return shard_q4(q, shard) if shard and shard.size > 1 else q
        t = fh.tensor(name)
        if info.dtype == "I8" and self.has(name + ".qb"):
            # block-32 int8 weights with a scale sidecar (the reference's optional Q8 weight format): served dense
            from .jq4 import q8_dequantize

            qb = name + ".qb"
            scales = self._files[self._where[qb]].tensor(qb).reshape(*info.shape[:-1], info.shape[-1] // BLOCK)
            t = q8_dequantize(t, scales.float(), torch.bfloat16)
        return shard_dense(t, shard) if shard and shard.size > 1 else t

    def load_dense(self, name: str, dtype: torch.dtype = torch.float32, shard: Optional[ShardSpec] = None) -> torch.Tensor:
        t = self.load(name, shard)
        if isinstance(t, Q4Tensor):
            return t.dequantize(dtype)
        return t.to(dtype)

    def close(self) -> None:
        for fh in self._files.values():
            fh.close()


def shard_dense(t: torch.Tensor, shard: ShardSpec) -> torch.Tensor:
    if shard.axis == "row":
        parts = [t[a:b] for a, b in shard.ranges(t.shape[0])]
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
    if shard.axis == "col":
        parts = [t[..., a:b] for a, b in shard.ranges(t.shape[-1])]
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=-1)
    raise ValueError(f"unknown shard axis {shard.axis}")


def shard_q4(q: Q4Tensor, shard: ShardSpec) -> Q4Tensor:
    shape = list(q.shape)
    if shard.axis == "row":
        rs = shard.ranges(shape[0])
        packed = torch.cat([q.packed[a:b] for a, b in rs], dim=0) if len(rs) > 1 else q.packed[rs[0][0] : rs[0][1]]
        scales = torch.cat([q.scales[a:b] for a, b in rs], dim=0) if len(rs) > 1 else q.scales[rs[0][0] : rs[0][1]]
        shape[0] = sum(b - a for a, b in rs)
        return Q4Tensor(packed, scales, tuple(shape))
    if shard.axis == "col":
        rs = shard.ranges(shape[-1])
        for a, b in rs:
            if a % BLOCK or b % BLOCK:
                raise ValueError(f"Q4 column shard [{a},{b}) is not aligned to the {BLOCK}-element block")
        packed = torch.cat([q.packed[..., a // 2 : b // 2] for a, b in rs], dim=-1)
        scales = torch.cat([q.scales[..., a // BLOCK : b // BLOCK] for a, b in rs], dim=-1)
        shape[-1] = sum(b - a for a, b in rs)
        return Q4Tensor(packed, scales, tuple(shape))
    raise ValueError(f"unknown shard axis {shard.axis}")
