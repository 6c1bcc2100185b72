"""Ragged batch description handed to a model forward: flattened tokens + per-sequence paged-KV metadata."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class ForwardBatch:
    token_ids: torch.Tensor  # [T] int32
    positions: torch.Tensor  # [T] int32
    slots: torch.Tensor  # [T] int64 flat cache rows (page * page_size + offset)
    q_start: torch.Tensor  # [S] int32 first row of each sequence
    q_len: torch.Tensor  # [S] int32 rows of each sequence in this step
    ctx_len: torch.Tensor  # [S] int32 cached tokens after this step
    block_tables: torch.Tensor  # [S, max_pages] int32
    is_decode: bool  # every sequence contributes exactly one row
    logits_rows: Optional[torch.Tensor] = None  # [S] int64 row of the last token of each sequence
    tile_seq: Optional[torch.Tensor] = None  # prefill tiling (64 query rows per tile)
    tile_q0: Optional[torch.Tensor] = None
    decode_splits: int = 1
    state_slots: Optional[torch.Tensor] = None  # [S] int64 recurrent-state slot per sequence (mamba layers)
    q_len_host: list = field(default_factory=list)
    ctx_len_host: list = field(default_factory=list)
    token_types: Optional[torch.Tensor] = None  # bert
    _tiles: dict = field(default_factory=dict)  # tile height -> (tile_seq, tile_q0) device tensors

    def tiles(self, rows: int):
        """Device tile arrays ``(tile_seq, tile_q0)`` for query tiles of ``rows`` rows (built once per height from ``q_len_host``)."""
        if rows == 64 and self.tile_seq is not None:
            return self.tile_seq, self.tile_q0
        got = self._tiles.get(rows)
        if got is None:
            from ..ops import prefill_tiles

            ts, t0 = prefill_tiles(list(self.q_len_host), rows)
            dev = self.q_len.device
            got = (torch.tensor(ts, dtype=torch.int32).to(dev, non_blocking=True), torch.tensor(t0, dtype=torch.int32).to(dev, non_blocking=True))
            self._tiles[rows] = got
        return got

    @property
    def num_tokens(self) -> int:
        return int(self.token_ids.shape[0])

    @property
    def num_seqs(self) -> int:
        return int(self.q_len.shape[0])


def make_batch(seqs: list[dict], page_size: int, device, max_pages: Optional[int] = None) -> ForwardBatch:
    """Build a batch from host-side sequence descriptions.

    Each entry: ``{"tokens": [new token ids], "start": first position, "pages": [page ids], "state_slot": int}``.
    """
    from ..ops import prefill_tiles

    toks, pos, slots, qs, ql, cl = [], [], [], [], [], []  # toks / pos / slots: one tensor per sequence
    width = max_pages or max(1, max(len(s["pages"]) for s in seqs))
    bt = torch.zeros(len(seqs), width, dtype=torch.int32)
    row = 0
    short: tuple[list, list, list] = ([], [], [])  # tokens / positions / slots of short sequences not yet turned into tensors

    def flush_short():
        if short[0]:
            toks.append(torch.tensor(short[0], dtype=torch.int32))
            pos.append(torch.tensor(short[1], dtype=torch.int32))
            slots.append(torch.tensor(short[2], dtype=torch.int64))
            for v in short:
                v.clear()

    for i, s in enumerate(seqs):
        n = len(s["tokens"])
        start = int(s["start"])
        pages = s["pages"]
        need = (start + n + page_size - 1) // page_size
        if need > len(pages):
            raise ValueError(f"sequence {i}: {need} pages needed, {len(pages)} given")
        pages_t = torch.tensor(pages, dtype=torch.int64)
        bt[i, : len(pages)] = pages_t
        qs.append(row)
        ql.append(n)
        cl.append(start + n)
        if n <= 16:  # decode rows and short tails: plain lists (a tensor op per sequence would cost more than the loop)
            for j in range(n):
                p = start + j
                short[0].append(int(s["tokens"][j]))
                short[1].append(p)
                short[2].append(pages[p // page_size] * page_size + p % page_size)
        else:
            # vectorised: a prompt chunk has thousands of tokens, and the device waits while the host builds the next chunk
            flush_short()
            p = torch.arange(start, start + n, dtype=torch.int64)
            toks.append(torch.as_tensor(s["tokens"], dtype=torch.int32))
            pos.append(p.to(torch.int32))
            slots.append(pages_t[p // page_size] * page_size + p % page_size)
        row += n
    flush_short()
    is_decode = all(n == 1 for n in ql)
    last = [a + b - 1 for a, b in zip(qs, ql)]
    ts, t0 = ([], []) if is_decode else prefill_tiles(ql)
    dev = torch.device(device)

    def t(v, dt):
        if v and isinstance(v[0], torch.Tensor):
            return torch.cat(v).to(dt).to(dev, non_blocking=True)
        return torch.tensor(v, dtype=dt).to(dev, non_blocking=True)

    state_slots = None
    if any("state_slot" in s for s in seqs):
        state_slots = t([int(s.get("state_slot", 0)) for s in seqs], torch.int64)
    return ForwardBatch(
        token_ids=t(toks, torch.int32), positions=t(pos, torch.int32), slots=t(slots, torch.int64), q_start=t(qs, torch.int32),
        q_len=t(ql, torch.int32), ctx_len=t(cl, torch.int32), block_tables=bt.to(dev, non_blocking=True), is_decode=is_decode,
        logits_rows=t(last, torch.int64), tile_seq=t(ts, torch.int32) if ts else None, tile_q0=t(t0, torch.int32) if ts else None,
        state_slots=state_slots, q_len_host=ql, ctx_len_host=cl,
    )
