"""Token sampling with the reference's order of operations, batched over the rows of a decode step.

Order (core/.../model/AbstractGeneratorSampler.java:100-323, ExcludeTopChoicePicker.java:42-86):
default ``top_p = 0.10`` when none of xtc/top_k/top_p/uniform_top_p is set; logits are scaled (Granite), soft-capped and
guided-masked upstream (:func:`deliverance_b200.ops.logits_post`); greedy = first maximum; XTC draws one uniform and, when
it fires, returns the least probable token above the threshold (or the most probable one if that is a special token);
otherwise ``sample_top_k_top_p``: scale by 1/T, stable descending sort, candidate limit (``top_k >= 1`` absolute, ``< 1``
fractional legacy: ``max(1, V - int(top_k * V))``), softmax over the kept set, smallest prefix whose cumulative mass reaches
``top_p``, then either a uniform pick inside that nucleus (``uniform_top_p``) or an inverse-CDF walk with
``pick = u * sum(exp)``. One uniform per sampled token (+ one per XTC attempt) from a per-request generator seeded with
``seed`` — deterministic per seed, not bit-identical to ``java.util.Random``.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..params import GeneratorParameters, TokenLogProb


@dataclass
class SamplingState:
    params: GeneratorParameters
    rng: random.Random = field(default_factory=lambda: random.Random(42))
    special_ids: frozenset = frozenset()

    @staticmethod
    def create(params: GeneratorParameters, special_ids=()) -> "SamplingState":
        return SamplingState(params, random.Random(params.seed), frozenset(special_ids))

    def effective(self):
        """(top_k, top_p, uniform_top_p, xtc_threshold, xtc_probability) after the reference's defaulting rule."""
        p = self.params
        top_k, top_p, utp = p.top_k, p.top_p, p.uniform_top_p
        xtc = p.xtc_threshold if p.xtc_threshold else None
        if xtc is None and top_k is None and top_p is None and utp is None:
            top_p = 0.10
        return top_k, top_p, utp, xtc, (p.xtc_probability if p.xtc_probability is not None else 0.0)

    @property
    def greedy(self) -> bool:
        return self.params.temperature == 0 and not self.params.xtc_threshold


def candidate_limit(top_k: Optional[float], V: int) -> int:
    if top_k is None:
        return V
    if top_k >= 1:
        return min(V, int(round(top_k)))
    return max(1, V - int(top_k * V))


def xtc_pick(logits_row: torch.Tensor, threshold: float, probability: float, u: float, special_ids) -> Optional[int]:
    """Exclude-top-choice: returns a token id or ``None`` when XTC does not fire."""
    if u > probability:
        return None
    probs = torch.softmax(logits_row.float(), dim=-1)
    above = torch.nonzero(probs > threshold).flatten()
    if above.numel() == 0:
        return None
    pa = probs[above]
    top = int(above[torch.argmax(pa)])
    if top in special_ids:
        return top
    return int(above[torch.argmin(pa)])


def sample_top_k_top_p_batch(logits: torch.Tensor, temps: torch.Tensor, limits: torch.Tensor, top_ps: torch.Tensor,
                             uniform: torch.Tensor, us: torch.Tensor) -> torch.Tensor:
    """Vectorised ``sampleTopKTopP`` over rows. ``top_ps <= 0`` means no nucleus cut. Returns token ids ``[B]``."""
    B, V = logits.shape
    scaled = logits.float() / temps.unsqueeze(1)
    vals, idx = torch.sort(scaled, dim=-1, descending=True, stable=True)
    ar = torch.arange(V, device=logits.device).unsqueeze(0)
    keep = ar < limits.unsqueeze(1)
    mx = vals[:, :1]
    ex = torch.where(keep, torch.exp(vals - mx), torch.zeros_like(vals))
    ex = torch.nan_to_num(ex, nan=0.0)
    total = ex.sum(dim=-1, keepdim=True)
    cum = torch.cumsum(ex, dim=-1)
    # nucleus: smallest prefix whose renormalised cumulative mass reaches top_p
    has_p = top_ps > 0
    target = torch.where(has_p, top_ps, torch.ones_like(top_ps)).unsqueeze(1) * total
    reach = cum >= target - 1e-12 * total
    n_p = torch.argmax(reach.to(torch.int8), dim=-1) + 1
    n_p = torch.where(reach.any(dim=-1), n_p, limits)
    n = torch.where(has_p, torch.minimum(n_p, limits), limits).clamp(min=1)
    # uniform pick inside the nucleus
    uni_idx = torch.minimum((us * n.float()).to(torch.int64), n - 1)
    # inverse-CDF walk: first i with cum[i] >= u * sum(exp over nucleus)
    nuc_total = torch.gather(cum, 1, (n - 1).unsqueeze(1))
    pick = us.unsqueeze(1) * nuc_total
    walk = (cum >= pick) & (ar < n.unsqueeze(1))
    walk_idx = torch.where(walk.any(dim=-1), torch.argmax(walk.to(torch.int8), dim=-1), n - 1)
    pos = torch.where(uniform, uni_idx, walk_idx)
    return torch.gather(idx, 1, pos.unsqueeze(1)).squeeze(1)


class Sampler:
    """Batched sampler. ``logits`` rows must already be scaled / soft-capped / guided-masked."""

    def __init__(self, decode_token=None):
        self.decode_token = decode_token or (lambda i: str(i))
        self.stats = {"kernel_rows": 0, "fallback_rows": 0}

    def _sample_cuda(self, logits: torch.Tensor, rest: list) -> list[int]:
        """Rows through the histogram-select kernel (csrc/sampling.cu); rows it declines (a histogram bin too crowded, a pick in
        the far tail) go through the sorting path. The per-row parameters travel as one pinned ``[6, n]`` float tensor (one
        host-to-device copy per step) and the picks come back with one read."""
        dev = logits.device
        n = len(rest)
        host = self._staging(n)
        host[0] = torch.tensor([r[0] for r in rest], dtype=torch.float32)
        host[1] = 1.0 / torch.tensor([r[1] for r in rest], dtype=torch.float32)
        host[2] = torch.tensor([min(r[2], 1 << 24) for r in rest], dtype=torch.float32)  # limits beyond 2^24 mean "the whole vocabulary"
        host[3] = torch.tensor([r[3] for r in rest], dtype=torch.float32)
        host[4] = torch.tensor([1.0 if r[4] else 0.0 for r in rest], dtype=torch.float32)
        host[5] = torch.tensor([r[5] for r in rest], dtype=torch.float32)
        packed = host.to(dev, non_blocking=True)
        res = ops.require_ext().sample_rows_packed(logits if logits.stride(1) == 1 else logits.contiguous(), packed).tolist()
        ops._count()
        tok_l, ok_l = res
        bad = [i for i, o in enumerate(ok_l) if not o]
        self.stats["kernel_rows"] += n - len(bad)
        self.stats["fallback_rows"] += len(bad)
        if bad:
            bi = torch.tensor(bad, device=dev)
            sub = logits if n == logits.shape[0] else logits.index_select(0, packed[0].to(torch.int64))
            fb = sample_top_k_top_p_batch(sub.index_select(0, bi), 1.0 / packed[1][bi], packed[2][bi].to(torch.int64), packed[3][bi],
                                          packed[4][bi] > 0, packed[5][bi]).tolist()
            for i, t in zip(bad, fb):
                tok_l[i] = t
        return [int(t) for t in tok_l]

    def _staging(self, n: int) -> torch.Tensor:
        """Pinned host staging for the packed sampling parameters (two buffers in turn: the copy of the previous step may still be in flight)."""
        bufs = self.__dict__.setdefault("_stage_bufs", {})
        turn = self.__dict__.get("_stage_turn", 0) ^ 1
        self.__dict__["_stage_turn"] = turn
        key = (n, turn)
        if key not in bufs:
            if len(bufs) > 64:
                bufs.clear()
            bufs[key] = torch.empty((6, n), dtype=torch.float32, pin_memory=torch.cuda.is_available())
        return bufs[key]

    def sample(self, logits: torch.Tensor, states: list[SamplingState]) -> tuple[list[int], list[Optional[TokenLogProb]]]:
        B, V = logits.shape
        out: list[Optional[int]] = [None] * B
        greedy_rows = [i for i, s in enumerate(states) if s.greedy]
        amax = None
        if greedy_rows or any(s.params.xtc_threshold for s in states):
            amax, _ = ops.argmax(logits)
        # XTC rows: one kernel for all of them on CUDA (csrc/sampling.cu::xtc_kernel), row by row with torch statements on the CPU
        rest = []
        xtc_rows = []
        for i, s in enumerate(states):
            if s.greedy:
                continue
            top_k, top_p, utp, xtc, xtc_prob = s.effective()
            T = s.params.temperature
            if xtc is not None:
                u = s.rng.random()
                if logits.device.type == "cuda":
                    xtc_rows.append((i, 1.0 if T == 0 else 1.0 / T, xtc, u <= xtc_prob, s.special_ids))
                    continue
                row = logits[i] if T == 0 else logits[i] / T
                pick = xtc_pick(row, xtc, xtc_prob, u, s.special_ids)
                out[i] = pick if pick is not None else int(amax[i])
                continue
            rest.append((i, T, candidate_limit(top_k, V), top_p if top_p is not None else 0.0, utp is not None, s.rng.random()))
        if xtc_rows:
            dev = logits.device
            sub = logits.index_select(0, torch.tensor([r[0] for r in xtc_rows], device=dev))
            special = sorted(set().union(*[r[4] for r in xtc_rows]))
            picks = ops.require_ext().xtc_rows(
                sub, torch.tensor([r[1] for r in xtc_rows], dtype=torch.float32, device=dev),
                torch.tensor([r[2] for r in xtc_rows], dtype=torch.float32, device=dev),
                torch.tensor([r[3] for r in xtc_rows], dtype=torch.uint8, device=dev),
                torch.tensor(special or [-1], dtype=torch.int32, device=dev)).tolist()
            ops._count()
            am = amax.tolist()
            for r, pk in zip(xtc_rows, picks):
                out[r[0]] = int(pk) if pk >= 0 else int(am[r[0]])
        if rest and logits.device.type == "cuda":
            toks = self._sample_cuda(logits, rest)
            for r, t in zip(rest, toks):
                out[r[0]] = int(t)
            rest = []
        if rest:
            rows = torch.tensor([r[0] for r in rest], device=logits.device)
            dev = logits.device
            toks = sample_top_k_top_p_batch(
                logits.index_select(0, rows),
                torch.tensor([r[1] for r in rest], dtype=torch.float32, device=dev),
                torch.tensor([r[2] for r in rest], dtype=torch.int64, device=dev),
                torch.tensor([r[3] for r in rest], dtype=torch.float32, device=dev),
                torch.tensor([r[4] for r in rest], dtype=torch.bool, device=dev),
                torch.tensor([r[5] for r in rest], dtype=torch.float32, device=dev),
            ).tolist()
            for r, t in zip(rest, toks):
                out[r[0]] = int(t)
        if greedy_rows:
            am = amax.tolist()
            for i in greedy_rows:
                out[i] = int(am[i])
        lps: list[Optional[TokenLogProb]] = [None] * B
        want = [i for i, s in enumerate(states) if s.params.logprobs]
        if want and logits.device.type == "cuda":
            # one kernel: log-sum-exp, the chosen token's log-probability and the top-N per row (csrc/sampling.cu::logprob_kernel)
            dev = logits.device
            sub = logits.index_select(0, torch.tensor(want, device=dev)).float()
            kmax = min(V, 64, max(states[i].params.top_logprobs for i in want))
            clp, topi, topv = ops.require_ext().logprob_rows(sub, torch.tensor([out[i] for i in want], dtype=torch.int64, device=dev), kmax)
            ops._count()
            clp, topi, topv = clp.tolist(), topi.tolist(), topv.tolist()
            for j, i in enumerate(want):
                tl = TokenLogProb(out[i], self.decode_token(out[i]), float(clp[j]))
                k = min(states[i].params.top_logprobs, kmax)
                if k > 0:
                    tl.top = [TokenLogProb(int(t), self.decode_token(int(t)), float(v)) for t, v in zip(topi[j][:k], topv[j][:k])]
                lps[i] = tl
        elif want:
            rows = torch.tensor(want, device=logits.device)
            sub = logits.index_select(0, rows).float()
            lse = torch.logsumexp(sub, dim=-1)
            chosen = torch.tensor([out[i] for i in want], device=logits.device)
            clp = (sub.gather(1, chosen.unsqueeze(1)).squeeze(1) - lse).tolist()
            kmax = max(states[i].params.top_logprobs for i in want)
            topv = topi = None
            if kmax > 0:
                topv, topi = torch.topk(sub, min(kmax, V), dim=-1)
                topv = (topv - lse.unsqueeze(1)).tolist()
                topi = topi.tolist()
            for j, i in enumerate(want):
                tl = TokenLogProb(out[i], self.decode_token(out[i]), float(clp[j]))
                k = states[i].params.top_logprobs
                if k > 0:
                    tl.top = [TokenLogProb(int(t), self.decode_token(int(t)), float(v)) for t, v in zip(topi[j][:k], topv[j][:k])]
                lps[i] = tl
        return [int(t) for t in out], lps
