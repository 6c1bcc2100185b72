"""Server configuration from a ``.properties`` file in the reference's key layout (or the same keys as JSON).

    python -m deliverance_b200.server --config qwen3-4b-jq4.properties [--models-root ~/.deliverance]

Keys (reference: web/src/main/java/net/deliverance/http/MultiModelProperties.java:58-135, web/*.properties,
tp_local/coordinator.properties; both ``model-name`` and ``modelName`` spellings occur in the reference's own files):

    server.port
    deliverance-model.configs[i].model-owner | model-name | model-dir       (model-dir: an explicit directory, extension)
    deliverance-model.configs[i].inference-type           GENERATION | EMBEDDING | CLASSIFICATION
    deliverance-model.configs[i].output-head-quantization Q4
    deliverance-model.configs[i].lora-adapter             adapter directory merged at load (extension)
    deliverance-model.configs[i].tensor-parallel.enabled | size
    deliverance.kv.prefix.max-tokens | checkpoint-policy | max-checkpoints | compression | turboquant.bits | enabled | max-entries
    deliverance.kv.context-rows-per-page-target | deliverance.kv.disk-dir
    deliverance.openai.reasoning-field                    openai | vllm
    deliverance.basic.auth.user | deliverance.basic.auth.password | deliverance.jwt.secret

Values may contain ``${NAME:default}`` placeholders resolved from the environment. Keys that only make sense for the
reference's runtime (``deliverance.tensor.operations.type``, gossip seeds / URIs, per-RPC timeouts) are accepted and listed in
``ignored``. A model is looked up as ``<models-root>/<owner>_<name>`` (the fetcher's cache layout), then ``<models-root>/<name>``.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Optional

_PLACEHOLDER = re.compile(r"\$\{([^}:]+)(?::([^}]*))?\}")
_INDEXED = re.compile(r"^deliverance-model\.configs\[(\d+)\]\.(.+)$")


def _kebab(key: str) -> str:
    """``modelName`` -> ``model-name`` (per dotted segment)."""
    return ".".join(re.sub(r"(?<=[a-z0-9])([A-Z])", lambda m: "-" + m.group(1).lower(), seg) for seg in key.split("."))


def parse_properties(text: str, env: Optional[dict] = None) -> dict:
    """Java ``.properties`` subset: ``key=value`` / ``key: value`` lines, ``#`` / ``!`` comments, trailing-backslash continuation."""
    env = os.environ if env is None else env
    out: dict = {}
    pending = ""
    for raw in text.splitlines():
        line = pending + raw.strip()
        pending = ""
        if not line or line[0] in "#!":
            continue
        if line.endswith("\\"):
            pending = line[:-1]
            continue
        m = re.match(r"([^=:\s]+)\s*[=:]\s*(.*)$", line) or re.match(r"(\S+)\s+(.*)$", line)
        if not m:
            out[line] = ""
            continue
        value = _PLACEHOLDER.sub(lambda p: env.get(p.group(1), p.group(2) if p.group(2) is not None else ""), m.group(2).strip())
        out[m.group(1)] = value
    return out


def _flatten(d: dict, prefix: str = "") -> dict:
    out = {}
    for k, v in d.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(_flatten(v, key + "."))
        elif isinstance(v, list) and all(isinstance(x, dict) for x in v):
            for i, x in enumerate(v):
                out.update(_flatten(x, f"{key}[{i}]."))
        else:
            out[key] = v if isinstance(v, str) else json.dumps(v) if isinstance(v, (list, dict)) else str(v)
    return out


@dataclass
class ModelEntry:
    owner: str = ""
    name: str = ""
    model_dir: str = ""
    inference_type: str = "GENERATION"
    output_head_quantization: Optional[str] = None
    lora_adapter: Optional[str] = None
    tp_enabled: bool = False
    tp_size: int = 0

    def resolve_dir(self, models_root: str) -> str:
        if self.model_dir:
            return os.path.expanduser(self.model_dir)
        root = os.path.expanduser(models_root)
        for cand in ((f"{self.owner}_{self.name}" if self.owner else None), self.name):
            if cand and os.path.isdir(os.path.join(root, cand)):
                return os.path.join(root, cand)
        return os.path.join(root, f"{self.owner}_{self.name}" if self.owner else self.name)


@dataclass
class ServerConfig:
    port: Optional[int] = None
    models: list = field(default_factory=list)
    kv: dict = field(default_factory=dict)  # KvCacheSettings field -> value
    kv_turboquant_bits: Optional[int] = None
    kv_disk_dir: Optional[str] = None  # evicted prefixes spill to files under this directory
    reasoning_field: Optional[str] = None
    basic_user: Optional[str] = None
    basic_password: Optional[str] = None
    jwt_secret: Optional[str] = None
    ignored: list = field(default_factory=list)

    def kv_settings(self):
        from ..kv.paged import KvCacheSettings

        return KvCacheSettings(**self.kv)


_KV_KEYS = {"deliverance.kv.prefix.max-tokens": ("max_prefix_tokens", int), "deliverance.kv.prefix.checkpoint-policy": ("policy", str.upper),
            "deliverance.kv.prefix.max-checkpoints": ("checkpoints", int), "deliverance.kv.prefix.compression": ("compression", str.upper),
            "deliverance.kv.prefix.enabled": ("enabled", lambda v: v.lower() == "true"), "deliverance.kv.prefix.max-entries": ("max_entries", int),
            "deliverance.kv.prefix.block-size": ("block_size", int), "deliverance.kv.context-rows-per-page-target": ("block_size", int)}


def load_server_config(path: str, env: Optional[dict] = None) -> ServerConfig:
    with open(path) as f:
        text = f.read()
    props = _flatten(json.loads(text)) if path.endswith(".json") else parse_properties(text, env)
    cfg = ServerConfig()
    entries: dict = {}
    for raw_key, v in props.items():
        key = _kebab(raw_key)
        m = _INDEXED.match(key)
        if m:
            e = entries.setdefault(int(m.group(1)), ModelEntry())
            sub = m.group(2)
            if sub == "model-owner":
                e.owner = v
            elif sub == "model-name":
                e.name = v
            elif sub == "model-dir":
                e.model_dir = v
            elif sub == "inference-type":
                e.inference_type = v.upper()
            elif sub == "output-head-quantization" or sub == "tensor-parallel.output-head-quantization":
                e.output_head_quantization = v or None
            elif sub == "lora-adapter":
                e.lora_adapter = v or None
            elif sub == "tensor-parallel.enabled":
                e.tp_enabled = v.lower() == "true"
            elif sub == "tensor-parallel.size":
                e.tp_size = int(v)
            else:
                cfg.ignored.append(raw_key)
        elif key in _KV_KEYS:
            name, conv = _KV_KEYS[key]
            cfg.kv[name] = conv(v)
        elif key == "deliverance.kv.prefix.turboquant.bits":
            cfg.kv_turboquant_bits = int(v)
        elif key == "deliverance.kv.disk-dir":
            cfg.kv_disk_dir = v or None
        elif key == "server.port":
            cfg.port = int(v)
        elif key == "deliverance.openai.reasoning-field":
            cfg.reasoning_field = v.lower()
        elif key == "deliverance.basic.auth.user":
            cfg.basic_user = v
        elif key == "deliverance.basic.auth.password":
            cfg.basic_password = v
        elif key == "deliverance.jwt.secret":
            cfg.jwt_secret = v
        else:
            cfg.ignored.append(raw_key)
    cfg.models = [entries[i] for i in sorted(entries)]
    for e in cfg.models:
        if e.inference_type not in ("GENERATION", "EMBEDDING", "CLASSIFICATION"):
            raise ValueError(f"unknown inference-type '{e.inference_type}' for model '{e.name}'")
        if not (e.name or e.model_dir):
            raise ValueError("a model entry needs model-name or model-dir")
    return cfg
