"""Disk tier of the prefix cache: evicted prefixes are written to files and pulled back into pages on a later hit.

The reference keeps evicted / cold KV pages in a disk backend that is a cache, not durable state (core/DiskKvBackend.md:6-12;
core/.../tensor/KvBufferCache.java ``kvbuffercache.disk.*`` counters). Here an evicted prefix entry (attention layers only)
is snapshotted with :func:`kv.turboquant.snapshot_pages` (``NONE`` | ``LZ4`` | ``MSE_TURBOQUANT``) into one safetensors file
(arrays plus a JSON header, nothing executable) named after the prefix key; a lookup that misses in memory probes the directory for the policy's checkpoint lengths, allocates pages,
restores the rows and re-registers the entry. Files are evicted oldest-first beyond ``max_bytes``.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from ..ckpt.safetensors_io import SafeTensorFile, write_safetensors
from .turboquant import Encoded, MseTurboQuantCodec, restore_pages, snapshot_pages


def _pack(snap: dict) -> tuple[dict, dict]:
    """Snapshot -> (tensors, metadata) for a safetensors file: nothing executable is stored, only arrays and a JSON header."""
    tensors, layers = {}, {}
    comp = snap["compression"]
    for i, (a, b) in snap["layers"].items():
        for tag, v in (("k", a), ("v", b)):
            name = f"l{i}.{tag}"
            if comp == "MSE_TURBOQUANT":
                tensors[name + ".codes"], tensors[name + ".norms"] = v.codes, v.norms
                layers[name] = {"shape": list(v.shape), "bits": v.bits}
            elif comp in ("LZ4", "DEFLATE"):
                raw, shape, dtype = v
                tensors[name] = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
                layers[name] = {"shape": list(shape), "dtype": str(dtype).replace("torch.", "")}
            else:
                tensors[name] = v.contiguous()
    codec = snap.get("codec")
    meta = {"compression": comp, "n_tokens": str(snap["n_tokens"]), "layers": json.dumps(layers), "layer_ids": json.dumps(sorted(snap["layers"])),
            "codec": json.dumps({"dim": codec.dim, "bits": codec.bits} if codec is not None else None)}
    return tensors, meta


def _unpack(f: SafeTensorFile) -> dict:
    meta = f.metadata
    comp = meta["compression"]
    info = json.loads(meta["layers"])
    codec_cfg = json.loads(meta["codec"])
    snap = {"compression": comp, "n_tokens": int(meta["n_tokens"]), "layers": {},
            "codec": MseTurboQuantCodec(codec_cfg["dim"], codec_cfg["bits"]) if codec_cfg else None}
    for i in json.loads(meta["layer_ids"]):
        pair = []
        for tag in ("k", "v"):
            name = f"l{i}.{tag}"
            if comp == "MSE_TURBOQUANT":
                pair.append(Encoded(f.tensor(name + ".codes").clone(), f.tensor(name + ".norms").clone(), tuple(info[name]["shape"]), info[name]["bits"]))
            elif comp in ("LZ4", "DEFLATE"):
                pair.append((f.tensor(name).numpy().tobytes(), tuple(info[name]["shape"]), getattr(torch, info[name]["dtype"])))
            else:
                pair.append(f.tensor(name).clone())
        snap["layers"][i] = tuple(pair)
    return snap


class DiskPrefixStore:
    def __init__(self, directory: str, compression: str = "LZ4", bits: int = 4, max_bytes: int = 8 << 30, max_age_s: float = 0.0):
        self.dir = directory
        self.compression = compression
        self.bits = bits
        self.max_bytes = max_bytes
        self.max_age_s = max_age_s  # files not read or written for this long are swept (0: keep until the byte limit evicts them)
        os.makedirs(directory, exist_ok=True)
        self.metrics = {"disk_writes": 0, "disk_hits": 0, "disk_misses": 0, "disk_evict": 0, "disk_bytes": 0}

    def _path(self, key: bytes) -> str:
        return os.path.join(self.dir, key.hex() + ".kv")

    def has(self, key: bytes) -> bool:
        return os.path.exists(self._path(key))

    def save(self, kv, key: bytes, pages: list[int], length: int) -> None:
        snap = snapshot_pages(kv, pages, length, self.compression, self.bits)
        tmp = self._path(key) + ".tmp"
        tensors, meta = _pack(snap)
        write_safetensors(tmp, tensors, meta)
        os.replace(tmp, self._path(key))
        self.metrics["disk_writes"] += 1
        self._trim()

    def load(self, kv, key: bytes) -> Optional[tuple[list[int], int]]:
        """Allocate pages and restore the prefix; returns (pages, length) holding one reference each, or None."""
        path = self._path(key)
        try:
            snap = _unpack(SafeTensorFile(path))
        except (OSError, ValueError, KeyError):
            self.metrics["disk_misses"] += 1
            return None
        n_pages = (snap["n_tokens"] + kv.page_size - 1) // kv.page_size
        if kv.allocator.available() < n_pages:
            self.metrics["disk_misses"] += 1
            return None
        pages = [kv.allocator.alloc() for _ in range(n_pages)]
        restore_pages(kv, snap, pages)
        os.utime(path, None)
        self.metrics["disk_hits"] += 1
        return pages, snap["n_tokens"]

    def sweep(self, now: Optional[float] = None) -> int:
        """Age sweeper: removes files whose last use (a hit refreshes the time stamp) is older than ``max_age_s``, and stale
        temporaries of writers that died. Runs on every write; callers may also run it periodically. Returns the number removed
        (the reference sweeps its disk pages by age in a background task, core/.../tensor/KvBufferCache.java:609-722)."""
        import time

        now = time.time() if now is None else now
        removed = 0
        for f in os.listdir(self.dir):
            p = os.path.join(self.dir, f)
            try:
                age = now - os.path.getmtime(p)
                if (f.endswith(".kv") and self.max_age_s > 0 and age > self.max_age_s) or (f.endswith(".tmp") and age > 600):
                    os.remove(p)
                    removed += 1
            except OSError:
                pass  # another process removed it first
        self.metrics["disk_evict"] += removed
        return removed

    def _trim(self) -> None:
        self.sweep()
        files = [(os.path.getmtime(os.path.join(self.dir, f)), os.path.getsize(os.path.join(self.dir, f)), os.path.join(self.dir, f))
                 for f in os.listdir(self.dir) if f.endswith(".kv")]
        total = sum(s for _, s, _ in files)
        for _, size, path in sorted(files):
            if total <= self.max_bytes:
                break
            os.remove(path)
            total -= size
            self.metrics["disk_evict"] += 1
        self.metrics["disk_bytes"] = total
