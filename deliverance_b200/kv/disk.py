"""Disk tier of the prefix cache: evicted prefixes are written to files and pulled back into pages on a later hit.

The reference keeps evicted / cold KV pages in a disk backend that is a cache, not durable state (core/DiskKvBackend.md:6-12;
core/.../tensor/KvBufferCache.java ``kvbuffercache.disk.*`` counters). Here an evicted prefix entry (attention layers only)
is snapshotted with :func:`kv.turboquant.snapshot_pages` (``NONE`` | ``LZ4`` | ``MSE_TURBOQUANT``) into one file named after
the prefix key; a lookup that misses in memory probes the directory for the policy's checkpoint lengths, allocates pages,
restores the rows and re-registers the entry. Files are evicted oldest-first beyond ``max_bytes``.
"""
from __future__ import annotations

import os
import pickle
from typing import Optional

from .turboquant import restore_pages, snapshot_pages


class DiskPrefixStore:
    def __init__(self, directory: str, compression: str = "LZ4", bits: int = 4, max_bytes: int = 8 << 30):
        self.dir = directory
        self.compression = compression
        self.bits = bits
        self.max_bytes = max_bytes
        os.makedirs(directory, exist_ok=True)
        self.metrics = {"disk_writes": 0, "disk_hits": 0, "disk_misses": 0, "disk_evict": 0, "disk_bytes": 0}

    def _path(self, key: bytes) -> str:
        return os.path.join(self.dir, key.hex() + ".kv")

    def has(self, key: bytes) -> bool:
        return os.path.exists(self._path(key))

    def save(self, kv, key: bytes, pages: list[int], length: int) -> None:
        snap = snapshot_pages(kv, pages, length, self.compression, self.bits)
        tmp = self._path(key) + ".tmp"
        with open(tmp, "wb") as f:
            pickle.dump(snap, f, protocol=pickle.HIGHEST_PROTOCOL)
        os.replace(tmp, self._path(key))
        self.metrics["disk_writes"] += 1
        self._trim()

    def load(self, kv, key: bytes) -> Optional[tuple[list[int], int]]:
        """Allocate pages and restore the prefix; returns (pages, length) holding one reference each, or None."""
        path = self._path(key)
        try:
            with open(path, "rb") as f:
                snap = pickle.load(f)
        except (OSError, pickle.UnpicklingError, EOFError):
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

    def _trim(self) -> None:
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
