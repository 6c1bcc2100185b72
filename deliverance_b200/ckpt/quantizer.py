"""Model-directory quantiser: HF safetensors checkpoint -> JQ4 checkpoint (``Q4`` entries + ``.qb`` sidecars).

Behaviour follows safetensors/.../ModelQuantizer.java: the default tensor filter (:48-98) quantises attention and MLP
projections, BERT encoder denses, Qwen-MoE / Mixtral expert projections, Granite shared/MoE/mamba projections (3-D stacked
tensors by last dim) and keeps embeddings, norms, ``lm_head`` and routers dense; only ``.weight`` tensors with
``cols % 32 == 0``; output shards ``model-%05d.safetensors`` + index, a ``deliverance-quantization.json`` manifest, a README
note and a ``.finished`` marker (:35-37,151-154,293,600-615). Quantise-on-demand builds into a staging directory and moves
it into place atomically; a directory with ``.finished`` is reused (core/.../model/AutoModelForCausaLm.java:624-658).
"""
from __future__ import annotations

import json
import os
import re
import shutil
import time
from typing import Callable, Optional

import torch

from .jq4 import BLOCK, q4_quantize
from .loader import WeightLoader
from .safetensors_io import Q4Tensor, write_sharded

MANIFEST = "deliverance-quantization.json"
FINISHED = ".finished"

_BERT = re.compile(r".*encoder\.layer\.\d+\.(attention\.self\.(query|key|value)|attention\.output\.dense|intermediate\.dense|output\.dense)\.weight$")
_QWEN_MOE = re.compile(r".*\.mlp\.experts\.\d+\.(gate_proj|up_proj|down_proj)\.weight$")
_MIXTRAL = re.compile(r".*\.block_sparse_moe\.experts\.\d+\.(w1|w2|w3)\.weight$")
_ATTN = tuple(f"self_attn.{n}_proj.weight" for n in "qkvo")
_MLP = tuple(f"mlp.{n}_proj.weight" for n in ("gate", "up", "down"))
_GRANITE = ("shared_mlp.input_linear.weight", "shared_mlp.output_linear.weight", "block_sparse_moe.input_linear.weight",
            "block_sparse_moe.output_linear.weight", "mamba.in_proj.weight", "mamba.out_proj.weight")


def DEFAULT_Q4_FILTER(name: str) -> bool:
    if name.endswith(".qb") or not name.endswith(".weight"):
        return False
    return (name.endswith(_ATTN) or name.endswith(_MLP) or name.endswith(_GRANITE) or bool(_BERT.match(name))
            or bool(_QWEN_MOE.match(name)) or bool(_MIXTRAL.match(name)))


def quantize_tensor(t: torch.Tensor, device: Optional[str] = None) -> Q4Tensor:
    """Quantise on ``device`` (the CUDA kernel is bit-exact with the host path) and return host tensors."""
    src = t.to(device) if device else t
    if src.device.type == "cuda":
        from .. import ops

        p, s = ops.q4_quantize(src.float())
        p, s = p.cpu(), s.cpu()
    else:
        p, s = q4_quantize(src)
    return Q4Tensor(p, s, tuple(t.shape))


class ModelQuantizer:
    def __init__(self, tensor_filter: Callable[[str], bool] = DEFAULT_Q4_FILTER, max_shard_bytes: int = 5 << 30,
                 device: Optional[str] = None):
        self.filter = tensor_filter
        self.max_shard_bytes = max_shard_bytes
        self.device = device

    def quantize(self, src_dir: str, out_dir: str) -> dict:
        loader = WeightLoader(src_dir)
        tensors: dict = {}
        changes = []
        for name in loader.names():
            info = loader.info(name)
            t = loader.load(name)
            if isinstance(t, Q4Tensor):
                tensors[name] = t
                continue
            if self.filter(name) and len(info.shape) >= 2 and info.shape[-1] % BLOCK == 0:
                tensors[name] = quantize_tensor(t, self.device)
                changes.append({"tensor": name, "from": info.dtype, "to": "Q4", "sidecar": name + ".qb", "shape": list(info.shape)})
            else:
                tensors[name] = t
        os.makedirs(out_dir, exist_ok=True)
        files = write_sharded(out_dir, tensors, self.max_shard_bytes, metadata={"format": "pt", "quantization": "JQ4"},
                              canonicalize_1d=True)
        for fname in os.listdir(src_dir):
            if fname.endswith(".safetensors") or fname == "model.safetensors.index.json" or fname in (MANIFEST, FINISHED):
                continue
            s = os.path.join(src_dir, fname)
            if os.path.isfile(s):
                shutil.copy2(s, os.path.join(out_dir, fname))
        manifest = {"source": os.path.abspath(src_dir), "output": os.path.abspath(out_dir), "format": "JQ4", "block_size": BLOCK,
                    "created": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "files": files, "tensors": changes}
        with open(os.path.join(out_dir, MANIFEST), "w") as f:
            json.dump(manifest, f, indent=1)
        with open(os.path.join(out_dir, "README.md"), "a") as f:
            f.write("\n\n## Quantization\n\nJQ4: packed 4-bit blocks of 32 with fp32 `.qb` scale sidecars; "
                    f"{len(changes)} tensors quantised.\n")
        with open(os.path.join(out_dir, FINISHED), "w") as f:
            f.write("ok\n")
        loader.close()
        return manifest


def quantize_on_demand(src_dir: str, target_dir: str, **kw) -> str:
    """Reuse ``target_dir`` when it carries ``.finished``; otherwise build in a staging directory and move into place."""
    if os.path.exists(os.path.join(target_dir, FINISHED)):
        return target_dir
    staging = target_dir.rstrip("/") + f".staging-{os.getpid()}"
    if os.path.exists(staging):
        shutil.rmtree(staging)
    ModelQuantizer(**kw).quantize(src_dir, staging)
    if os.path.exists(target_dir):
        shutil.rmtree(target_dir)
    os.replace(staging, target_dir)
    return target_dir


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Quantise a HF safetensors model directory to JQ4")
    ap.add_argument("src")
    ap.add_argument("out")
    ap.add_argument("--device", default=None)
    ap.add_argument("--max-shard-gb", type=float, default=5.0)
    a = ap.parse_args(argv)
    m = ModelQuantizer(max_shard_bytes=int(a.max_shard_gb * (1 << 30)), device=a.device).quantize(a.src, a.out)
    print(f"quantised {len(m['tensors'])} tensors into {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
