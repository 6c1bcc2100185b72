"""Paged KV pool with a block-hash prefix cache that shares pages by reference count.

Semantics kept from the reference's ``KvBufferCache`` (core/.../tensor/KvBufferCache.java:129-143,256-298,457-507;
core/PrefixCache.md:45-84): the key of a cached prefix is ``(salt, exact token prefix)``; hits happen only at multiples of
the block size (32 tokens); the probed/stored lengths follow a checkpoint policy (``FIXED_BLOCKS`` = every multiple,
``START_AND_END`` = ``{32, 64, L-32, L}``, ``ANCHORS`` = 32/64/128-aligned anchors + L); lookup returns the longest hit; a
full-prompt hit replays the last prompt token; entries are evicted LRU beyond ``max_entries``. Salts compose as
``cache_salt`` -> ``lora:<id>|salt`` -> ``tp:size=N:rank=R|...`` (LocalGenerationBackend.java:36-50,
InProcessTensorParallelRankService.java:96-103).

What differs by design: the reference copies a full KV snapshot per checkpoint; here a prefix is a chain of page ids
whose reference counts are bumped, so a hit costs no copy and no extra memory, and the 512-token cap
(``max_prefix_tokens``) is a setting, not a limit of the data structure.

Layout per attention layer: ``k[pages, KV, page_size, D]`` and ``v[...]`` in the working dtype; page 0 is a scratch page
that padded batch rows write to. Recurrent (mamba) layers get per-sequence state slots instead of pages.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional

import torch

PAGE_SIZE = 32


@dataclass
class KvCacheSettings:
    """Defaults follow core/.../tensor/KvBufferCacheSettings.java:20-31,45 (block 32, 512 prefix tokens, 10,000 entries)."""

    block_size: int = PAGE_SIZE
    max_prefix_tokens: int = 512
    max_entries: int = 10_000
    policy: str = "START_AND_END"  # FIXED_BLOCKS | START_AND_END | ANCHORS_AND_LARGEST
    checkpoints: int = 4  # most checkpoints kept per prompt (START_AND_END, ANCHORS_AND_LARGEST)
    anchors: tuple = (32, 64, 128)
    enabled: bool = True
    compression: str = "NONE"  # NONE | LZ4 | DEFLATE | MSE_TURBOQUANT (host snapshots only, see kv.turboquant)

    def checkpoint_lengths(self, n_tokens: int) -> list[int]:
        """Prefix lengths (multiples of the block size, at most ``max_prefix_tokens``) at which a prompt of ``n_tokens`` is
        checkpointed (reference: core/.../tensor/KvBufferCache.java:457-507 and the vectors of KvBufferCachePrefixTest.java):
        FIXED_BLOCKS = every block; START_AND_END = the first ceil(checkpoints / 2) blocks and the last floor(checkpoints / 2)
        block ends; ANCHORS_AND_LARGEST = the anchors that fit (at most checkpoints - 1 of them) plus the largest aligned length."""
        b = self.block_size
        L = (min(n_tokens, self.max_prefix_tokens) // b) * b
        if L < b:
            return []
        if self.policy == "FIXED_BLOCKS":
            return list(range(b, L + 1, b))
        m = max(1, self.checkpoints)
        if self.policy == "START_AND_END":
            n_start = (m + 1) // 2
            n_end = m - n_start
            picked = set(range(b, min(L, n_start * b) + 1, b))
            picked.update(x for x in range(L - (n_end - 1) * b, L + 1, b) if x >= b)
            return sorted(picked)
        if self.policy in ("ANCHORS_AND_LARGEST", "ANCHORS"):
            picked: list = []
            for a in self.anchors:
                a = (a // b) * b
                if b <= a <= L and a not in picked:
                    picked.append(a)
                if len(picked) >= max(0, m - 1):
                    break
            out = sorted(set(picked) | {L})
            return sorted(set(out[: m - 1] + [L])) if len(out) > m else out
        raise ValueError(f"unknown checkpoint policy {self.policy}")


class PageAllocator:
    """Free list + reference counts over page ids ``1 .. num_pages - 1`` (page 0 is scratch)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free = list(range(num_pages - 1, 0, -1))
        self.ref = [0] * num_pages

    def available(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("KV cache is out of pages")
        p = self.free.pop()
        self.ref[p] = 1
        return p

    def retain(self, p: int) -> None:
        self.ref[p] += 1

    def release(self, p: int) -> None:
        self.ref[p] -= 1
        if self.ref[p] == 0:
            self.free.append(p)
        elif self.ref[p] < 0:
            raise RuntimeError(f"page {p} released more often than retained")


@dataclass
class PrefixEntry:
    pages: list[int]
    length: int
    state: Optional[dict] = None  # recurrent-state snapshot for hybrid models


class PrefixCache:
    """LRU map ``hash(salt, tokens[:L]) -> pages`` holding one reference per cached page."""

    def __init__(self, settings: KvCacheSettings, allocator: PageAllocator):
        self.settings = settings
        self.alloc = allocator
        self.entries: "OrderedDict[bytes, PrefixEntry]" = OrderedDict()
        self.metrics = {"lookup": 0, "hits": 0, "misses": 0, "evict": 0, "stored": 0, "hit_tokens": 0}
        self.disk = None  # optional second tier (kv.disk.DiskPrefixStore), attached by PagedKVCache.attach_disk
        self.kv = None
        self.held: dict = {}  # page -> number of cache entries that hold a reference to it

    def _count(self, pages: list, d: int) -> None:
        held = self.held
        for p in pages:
            n = held.get(p, 0) + d
            if n > 0:
                held[p] = n
            else:
                held.pop(p, None)

    def reclaimable(self, want: int) -> int:
        """How many pages (counted up to ``want``) evicting cache entries would really free: pages that nothing but cache
        entries hold (entries of several checkpoint lengths share pages; running sequences that hit the cache hold them too)."""
        ref, n = self.alloc.ref, 0
        for p, c in self.held.items():
            if ref[p] == c:
                n += 1
                if n >= want:
                    break
        return n

    @staticmethod
    def key(salt: str, tokens: list[int]) -> bytes:
        h = hashlib.blake2b(digest_size=20)
        h.update(salt.encode("utf-8"))
        h.update(b"\x00")
        h.update(torch.tensor(tokens, dtype=torch.int64).numpy().tobytes())
        return h.digest()

    def lookup(self, salt: str, tokens: list[int]) -> Optional[PrefixEntry]:
        """Longest cached prefix among the policy's checkpoint lengths (retains its pages for the caller)."""
        self.metrics["lookup"] += 1
        if not self.settings.enabled:
            self.metrics["misses"] += 1
            return None
        best = None
        for L in sorted(self.settings.checkpoint_lengths(len(tokens)), reverse=True):
            k = self.key(salt, tokens[:L])
            e = self.entries.get(k)
            if e is not None:
                self.entries.move_to_end(k)
                best = e
                break
        if best is None and self.disk is not None:
            for L in sorted(self.settings.checkpoint_lengths(len(tokens)), reverse=True):
                k = self.key(salt, tokens[:L])
                if self.disk.has(k):
                    got = self.disk.load(self.kv, k)
                    if got is not None:
                        best = PrefixEntry(got[0], got[1], None)
                        self.entries[k] = best  # the entry owns the references taken by load()
                        self._count(best.pages, +1)
                        break
        if best is None:
            self.metrics["misses"] += 1
            return None
        self.metrics["hits"] += 1
        self.metrics["hit_tokens"] += best.length
        for p in best.pages:
            self.alloc.retain(p)
        return PrefixEntry(list(best.pages), best.length, best.state)

    def store(self, salt: str, tokens: list[int], pages: list[int], state_at: Optional[dict] = None) -> int:
        """Register the checkpoint prefixes of a prompt whose KV now lives in ``pages``. Returns entries added."""
        if not self.settings.enabled:
            return 0
        added = 0
        b = self.settings.block_size
        for L in self.settings.checkpoint_lengths(len(tokens)):
            k = self.key(salt, tokens[:L])
            if k in self.entries:
                self.entries.move_to_end(k)
                continue
            if state_at is not None and L not in state_at:
                continue  # hybrid models can only resume where a recurrent-state snapshot exists
            chain = pages[: L // b]
            for p in chain:
                self.alloc.retain(p)
            self.entries[k] = PrefixEntry(list(chain), L, None if state_at is None else state_at[L])
            self._count(chain, +1)
            added += 1
            self.metrics["stored"] += 1
        while len(self.entries) > self.settings.max_entries:
            self.evict_one()
        return added

    def evict_one(self) -> bool:
        if not self.entries:
            return False
        k, e = self.entries.popitem(last=False)
        if self.disk is not None and e.state is None and not self.disk.has(k):
            self.disk.save(self.kv, k, e.pages, e.length)  # spill before the pages go back to the allocator
        self._count(e.pages, -1)
        for p in e.pages:
            self.alloc.release(p)
        self.metrics["evict"] += 1
        return True

    def clear(self) -> None:
        while self.evict_one():
            pass


class PagedKVCache:
    """Device storage + allocator + prefix cache for one model replica (one tensor-parallel rank)."""

    def __init__(self, layout: dict, num_pages: int, device, dtype, settings: Optional[KvCacheSettings] = None,
                 max_state_slots: int = 0, mamba_shapes: Optional[dict] = None):
        self.settings = settings or KvCacheSettings()
        self.page_size = self.settings.block_size
        if self.page_size % 32:
            raise ValueError("page size must be a multiple of 32")
        self.device = torch.device(device)
        self.dtype = dtype
        self.num_pages = num_pages
        self.layout = layout
        kinds = layout["layer_kinds"]
        self.k: list[Optional[torch.Tensor]] = []
        self.v: list[Optional[torch.Tensor]] = []
        # optional per-layer shapes and cache sharing (gemma4: wide global heads, late layers reuse an earlier layer's cache)
        heads = layout.get("kv_heads_per_layer") or [layout["kv_heads"]] * len(kinds)
        dims = layout.get("head_dim_per_layer") or [layout["head_dim"]] * len(kinds)
        shared = layout.get("shared_from") or [-1] * len(kinds)
        for i, kind in enumerate(kinds):
            if kind == "mamba":
                self.k.append(None)
                self.v.append(None)
            elif shared[i] >= 0:
                self.k.append(self.k[shared[i]])
                self.v.append(self.v[shared[i]])
            else:
                shape = (num_pages, heads[i], self.page_size, dims[i])
                self.k.append(torch.zeros(shape, dtype=dtype, device=self.device))
                self.v.append(torch.zeros(shape, dtype=dtype, device=self.device))
        self.allocator = PageAllocator(num_pages)
        self.prefix = PrefixCache(self.settings, self.allocator)
        self.prefix.kv = self
        # recurrent state (hybrid models): per layer conv_state [slots, convDim, K-1] and ssm_state [slots, H, d_head, S]
        self.conv_state: dict[int, torch.Tensor] = {}
        self.ssm_state: dict[int, torch.Tensor] = {}
        self.free_slots = list(range(max_state_slots - 1, -1, -1))
        if mamba_shapes and max_state_slots > 0:
            for i, kind in enumerate(kinds):
                if kind == "mamba":
                    self.conv_state[i] = torch.zeros((max_state_slots,) + tuple(mamba_shapes["conv"]), dtype=torch.float32, device=self.device)
                    self.ssm_state[i] = torch.zeros((max_state_slots,) + tuple(mamba_shapes["ssm"]), dtype=torch.float32, device=self.device)

    def layer(self, i: int):
        return self.k[i], self.v[i]

    @staticmethod
    def bytes_per_page(layout: dict, page_size: int, dtype) -> int:
        kinds = layout["layer_kinds"]
        heads = layout.get("kv_heads_per_layer") or [layout["kv_heads"]] * len(kinds)
        dims = layout.get("head_dim_per_layer") or [layout["head_dim"]] * len(kinds)
        shared = layout.get("shared_from") or [-1] * len(kinds)
        rows = sum(heads[i] * dims[i] for i, k in enumerate(kinds) if k != "mamba" and shared[i] < 0)
        return 2 * rows * page_size * torch.empty((), dtype=dtype).element_size()

    # -- per-sequence page management ---------------------------------------------------------------------------
    def ensure_pages(self, pages: list[int], n_tokens: int) -> None:
        need = (n_tokens + self.page_size - 1) // self.page_size
        while len(pages) < need:
            if self.allocator.available() == 0 and not self.prefix.evict_one():
                raise MemoryError("KV cache is out of pages")
            if self.allocator.available() == 0:
                continue
            pages.append(self.allocator.alloc())

    def release_pages(self, pages: list[int]) -> None:
        for p in pages:
            self.allocator.release(p)
        pages.clear()

    def can_allocate(self, n_pages: int) -> bool:
        """True when ``n_pages`` can be had from the free list plus what evicting prefix-cache entries would really free:
        a cached page comes back only if nothing but cache entries holds it (entries of several checkpoint lengths share
        pages, and running sequences that hit the cache hold references too)."""
        free = self.allocator.available()
        return free >= n_pages or free + self.prefix.reclaimable(n_pages - free) >= n_pages

    def audit(self, sequences) -> None:
        """Consistency check for tests and debugging: every page's reference count must equal the number of sequences that list
        it plus the number of prefix-cache entries that hold it; free pages have count 0 and are listed once; page 0 (scratch)
        is never handed out. ``sequences``: iterables of page ids (the running requests' page lists). Raises AssertionError."""
        want = [0] * self.num_pages
        for pages in sequences:
            for p in pages:
                want[p] += 1
        per_entry: dict = {}
        for e in self.prefix.entries.values():
            for p in e.pages:
                want[p] += 1
                per_entry[p] = per_entry.get(p, 0) + 1
        assert per_entry == self.prefix.held, "prefix-cache holder counts out of date"
        free = self.allocator.free
        assert len(set(free)) == len(free) and 0 not in free, "free list has duplicates or the scratch page"
        for p in range(1, self.num_pages):
            assert self.allocator.ref[p] == want[p], f"page {p}: reference count {self.allocator.ref[p]}, holders {want[p]}"
            assert (want[p] == 0) == (p in free) or want[p] > 0, f"page {p}: free-list membership does not match its count"
        assert sum(1 for p in range(1, self.num_pages) if want[p] == 0) == len(free), "free page count mismatch"

    def alloc_state_slot(self) -> int:
        if not self.free_slots:
            raise MemoryError("no free recurrent-state slot")
        s = self.free_slots.pop()
        for t in list(self.conv_state.values()) + list(self.ssm_state.values()):
            t[s].zero_()
        return s

    def free_state_slot(self, s: int) -> None:
        self.free_slots.append(s)

    def snapshot_state(self, slot: int) -> dict:
        return {"conv": {i: t[slot].clone() for i, t in self.conv_state.items()},
                "ssm": {i: t[slot].clone() for i, t in self.ssm_state.items()}}

    def restore_state(self, slot: int, snap: dict) -> None:
        for i, t in snap["conv"].items():
            self.conv_state[i][slot].copy_(t)
        for i, t in snap["ssm"].items():
            self.ssm_state[i][slot].copy_(t)

    def attach_disk(self, directory: str, compression: str = "LZ4", bits: int = 4, max_bytes: int = 8 << 30, max_age_s: float = 0.0):
        """Spill evicted prefixes to ``directory`` and pull them back on later hits (attention-only models)."""
        from .disk import DiskPrefixStore

        self.prefix.disk = DiskPrefixStore(directory, compression, bits, max_bytes, max_age_s)
        return self.prefix.disk

    def gather_rows(self, layer: int, pages: list[int], n_tokens: int):
        """Dense ``[KV, n_tokens, D]`` copies of K and V (tests, snapshots, debugging)."""
        idx = torch.tensor(pages[: (n_tokens + self.page_size - 1) // self.page_size], device=self.device, dtype=torch.long)
        kh, hd = self.k[layer].shape[1], self.k[layer].shape[3]
        k = self.k[layer][idx].permute(1, 0, 2, 3).reshape(kh, -1, hd)[:, :n_tokens]
        v = self.v[layer][idx].permute(1, 0, 2, 3).reshape(kh, -1, hd)[:, :n_tokens]
        return k, v


def compose_salt(cache_salt: str = "", lora_id: Optional[str] = None, tp_rank: int = 0, tp_size: int = 1) -> str:
    salt = cache_salt or ""
    if lora_id:
        salt = f"lora:{lora_id}|{salt}"
    if tp_size > 1:
        salt = f"tp:size={tp_size}:rank={tp_rank}|{salt}"
    return salt
