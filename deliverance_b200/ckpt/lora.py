"""LoRA / PEFT adapters: load, merge into dense bases at load time, and runtime hot-swap deltas.

Adapter directory = ``adapter_config.json`` (``r``, ``lora_alpha``, ``target_modules``; other keys ignored) +
``adapter_model.safetensors`` with tensors ``base_model.model.<base-without-.weight>.lora_{A,B}.weight``; A ``[r, in]``,
B ``[out, r]``; merge ``W' = W + (alpha / r) * B @ A`` for dense bases only and not under tensor parallelism; hot-swap
keeps A and the pre-scaled B and adds ``(x @ A^T) @ (scale * B)^T`` at run time (reference: safetensors/.../
LoraAdapterConfig.java:21-54, LoraTensorNames.java:18-56, MergingWeightLoader.java:30-141, ResolvedLoraAdapter.java:22-45,
core/.../generator/LoraDeltaApplier.java:43-63).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from .loader import ShardSpec, WeightLoader
from .safetensors_io import Q4Tensor, SafeTensorFile

PREFIX = "base_model.model."


def lora_names(base_tensor: str) -> tuple[str, str]:
    """``model.layers.0.self_attn.q_proj.weight`` -> its lora_A / lora_B tensor names."""
    stem = base_tensor[: -len(".weight")] if base_tensor.endswith(".weight") else base_tensor
    return f"{PREFIX}{stem}.lora_A.weight", f"{PREFIX}{stem}.lora_B.weight"


def base_name(lora_tensor: str) -> Optional[str]:
    if not lora_tensor.startswith(PREFIX):
        return None
    for suf in (".lora_A.weight", ".lora_B.weight"):
        if lora_tensor.endswith(suf):
            return lora_tensor[len(PREFIX) : -len(suf)] + ".weight"
    return None


@dataclass
class LoraAdapterConfig:
    r: int
    lora_alpha: float
    target_modules: list = field(default_factory=list)

    @property
    def scale(self) -> float:
        return float(self.lora_alpha) / float(self.r)

    @staticmethod
    def load(path: str) -> "LoraAdapterConfig":
        with open(path) as f:
            d = json.load(f)
        if "r" not in d or "lora_alpha" not in d:
            raise ValueError("adapter_config.json needs 'r' and 'lora_alpha'")
        tm = d.get("target_modules") or []
        return LoraAdapterConfig(int(d["r"]), float(d["lora_alpha"]), [tm] if isinstance(tm, str) else list(tm))


class LoraAdapter:
    def __init__(self, adapter_dir: str, adapter_id: Optional[str] = None):
        self.dir = adapter_dir
        self.id = adapter_id or os.path.basename(os.path.normpath(adapter_dir))
        self.config = LoraAdapterConfig.load(os.path.join(adapter_dir, "adapter_config.json"))
        self.file = SafeTensorFile(os.path.join(adapter_dir, "adapter_model.safetensors"))
        self.pairs: dict[str, tuple[str, str]] = {}
        names = set(self.file.names())
        for n in names:
            b = base_name(n)
            if b is None:
                continue
            a_name, b_name = lora_names(b)
            if a_name in names and b_name in names:
                self.pairs[b] = (a_name, b_name)

    def targets(self) -> list[str]:
        return sorted(self.pairs)

    def has(self, base_tensor: str) -> bool:
        return base_tensor in self.pairs

    def ab(self, base_tensor: str) -> tuple[torch.Tensor, torch.Tensor]:
        a_name, b_name = self.pairs[base_tensor]
        A, B = self.file.tensor(a_name).float(), self.file.tensor(b_name).float()
        if A.shape[0] != self.config.r or B.shape[1] != self.config.r:
            raise ValueError(f"{base_tensor}: adapter rank mismatch (A {tuple(A.shape)}, B {tuple(B.shape)}, r={self.config.r})")
        return A, B

    def delta(self, base_tensor: str) -> torch.Tensor:
        A, B = self.ab(base_tensor)
        return self.config.scale * (B @ A)

    def resolved(self, base_tensor: str) -> tuple[torch.Tensor, torch.Tensor]:
        """(A, scale * B) for run-time application."""
        A, B = self.ab(base_tensor)
        return A, B * self.config.scale


class MergingWeightLoader(WeightLoader):
    """A weight loader that adds ``(alpha/r) * B @ A`` to every dense base tensor targeted by the adapter."""

    def __init__(self, model_dir: str, adapter: LoraAdapter):
        super().__init__(model_dir)
        self.adapter = adapter

    def load(self, name: str, shard: Optional[ShardSpec] = None):
        if not self.adapter.has(name):
            return super().load(name, shard)
        if shard is not None and shard.size > 1:
            raise ValueError("LoRA merge is not supported under tensor parallelism")
        base = super().load(name, None)
        if isinstance(base, Q4Tensor):
            raise ValueError(f"LoRA merge needs a dense base tensor, '{name}' is Q4")
        d = self.adapter.delta(name)
        if d.shape != base.shape:
            raise ValueError(f"{name}: delta shape {tuple(d.shape)} does not match base {tuple(base.shape)}")
        return (base.float() + d).to(base.dtype)


def apply_lora_delta(x: torch.Tensor, y: torch.Tensor, a: torch.Tensor, b_scaled: torch.Tensor) -> torch.Tensor:
    """``y + (x @ A^T) @ (scale*B)^T``. On CUDA (bf16, rank <= 64) one kernel adds the delta into ``y`` in place
    (csrc/aux.cu::lora_delta_kernel); elsewhere two skinny matrix products and an add."""
    if (y.is_cuda and y.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and a.dtype == torch.bfloat16 and b_scaled.dtype == torch.bfloat16
            and a.shape[0] <= 64 and x.dim() == 2 and y.dim() == 2 and x.stride(1) == 1 and y.stride(1) == 1 and x.shape[1] % 2 == 0 and x.stride(0) % 2 == 0):
        from .. import ops

        ops.require_ext().lora_delta(x, a.contiguous(), b_scaled.contiguous(), y)
        ops._count()
        return y
    t = x.to(a.dtype) @ a.t()
    return (y.to(a.dtype) + t @ b_scaled.t()).to(y.dtype)
