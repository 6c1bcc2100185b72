"""Continuous-batching generation engine.

The reference runs one independent ``generate`` loop per request (core/.../model/GenerationEngine.java:81-176; no request
batching, web/.../ChatCompletionController.java:373-383). Here one engine owns the model replica, the paged KV pool and
all in-flight requests: every :meth:`Engine.step` is either a chunked-prefill step over waiting requests or one decode
step over every running request (captured in a CUDA graph per batch-size bucket on GPUs). Per-request behaviour is kept:
prompt-length check against ``ntokens`` (GenerationEngine.java:98-104), prefix-cache lookup/store with salted keys, replay
of the last prompt token on a full-prompt hit (GenerationCursor.java:40-60), TTFT/throughput accounting (:249-268), and the
stop order max_tokens -> guided-choice complete -> stop strings -> tool-parser end of turn -> EOS (:189-219).
"""
from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .. import ops
from ..kv.paged import KvCacheSettings, PagedKVCache, compose_salt
from ..models.batch import ForwardBatch, make_batch
from ..params import FinishReason, GeneratorParameters, Response, TokenLogProb
from .sampler import Sampler, SamplingState

_log = logging.getLogger("deliverance_b200.engine")

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    rid: int
    prompt: list[int]
    params: GeneratorParameters
    on_token: Optional[Callable[[int, "Request"], None]] = None
    state: str = WAITING
    pages: list[int] = field(default_factory=list)
    computed: int = 0  # tokens whose KV is in the cache
    output: list[int] = field(default_factory=list)
    logprobs: list[TokenLogProb] = field(default_factory=list)
    sampling: Optional[SamplingState] = None
    guide: object = None  # guided-decoding logits processor (allowed-mask provider)
    stopper: object = None  # text-level stop detector (stop strings, tool parser)
    finish_reason: Optional[FinishReason] = None
    prefix_hit: int = 0
    state_slot: int = -1
    salt: str = ""
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    limit: int = 0  # absolute position limit
    cancelled: bool = False
    pending: int = 0  # tokens launched on the device but not yet read by the host (lookahead decode)
    error: Optional[str] = None
    state_snapshots: dict = field(default_factory=dict)
    fill: Optional[list] = None  # tokens whose KV must be cached before decoding: the prompt, or after a preemption prompt + output[:-1]
    resumed: bool = False  # re-admitted after a preemption: the prefill only rebuilds the cache, nothing is sampled from it
    preemptions: int = 0
    t_progress: float = 0.0

    def __post_init__(self):
        if self.fill is None:
            self.fill = self.prompt

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    def response(self) -> Response:
        r = Response()
        r.token_ids = list(self.output)
        r.prompt_tokens = len(self.prompt)
        r.generated_tokens = len(self.output)
        r.finish_reason = self.finish_reason or FinishReason.MAX_TOKENS
        r.sampler_returns = list(self.logprobs)
        r.ttft_ms = (self.t_first - self.t_submit) * 1e3 if self.t_first else 0.0
        r.total_ms = ((self.t_done or time.perf_counter()) - self.t_submit) * 1e3
        r.avg_ms_per_token = r.total_ms / max(1, r.generated_tokens)
        r.prefix_hit_tokens = self.prefix_hit
        return r


@dataclass
class EngineConfig:
    max_batch_tokens: int = 8192  # prefill token budget per step (the reference chunks prompts at 512, AbstractModel.java:87)
    max_seqs: int = 128
    num_pages: Optional[int] = None  # default: sized from free device memory
    kv_memory_fraction: float = 0.85
    cuda_graphs: bool = True
    device_timeout_s: float = 120.0  # watchdog of the lookahead path: a step that does not finish in this time raises
    lookahead: bool = True  # overlap the host bookkeeping of step N with the device work of step N + 1 (greedy graph decode)
    # 0: prefill work always goes first (best time to first token, running sequences wait while prompts are computed);
    # k > 0: after k consecutive prefill steps one decode step runs for the sequences that are ready (bounded inter-token latency)
    decode_interleave: int = 0
    kv: KvCacheSettings = field(default_factory=KvCacheSettings)
    max_state_slots: int = 0


_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class Engine:
    def __init__(self, model, config: Optional[EngineConfig] = None, eos_ids=(), special_ids=(), decode_token=None):
        self.model = model
        self.cfg = model.cfg
        self.config = config or EngineConfig()
        self.device = model.device
        self.eos_ids = frozenset(eos_ids or self.cfg.eos_token_ids)
        self.special_ids = frozenset(special_ids)
        self.sampler = Sampler(decode_token)
        layout = model.kv_layout()
        pages = self.config.num_pages or self._auto_pages(layout)
        tp = getattr(model, "tp", None)
        if self.config.num_pages is None and tp is not None and tp.enabled and tp.collectives is not None:
            # ranks size their pools from their own free memory; admission and preemption must decide alike on every rank
            # (a rank with a smaller pool would run a different batch and the collectives would no longer match): take the minimum
            mine = torch.tensor([float(pages)], dtype=torch.float32, device=self.device)
            pages = int(min(float(t.item()) for t in tp.collectives.all_gather(mine)))
        mamba_shapes = None
        slots = self.config.max_state_slots
        if any(k == "mamba" for k in layout["layer_kinds"]):
            c = self.cfg
            mamba_shapes = {"conv": (c.mamba_conv_dim, c.mamba_d_conv - 1), "ssm": (c.mamba_n_heads, c.mamba_d_head, c.mamba_d_state)}
            slots = slots or self.config.max_seqs
        self.kv = PagedKVCache(layout, pages, self.device, model.dtype, self.config.kv, slots, mamba_shapes)
        self.page_size = self.kv.page_size
        self.max_pages_per_seq = (self.cfg.max_position_embeddings + self.page_size - 1) // self.page_size
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self._next_id = 0
        self._graphs: dict[int, dict] = {}
        self._failed: list[Request] = []  # requests failed inside a step (reported by step())
        self._prefill_streak = 0
        self.metrics = {"steps": 0, "prefill_steps": 0, "decode_steps": 0, "prefill_tokens": 0, "decode_tokens": 0,
                        "graph_replays": 0, "kernel_launches": 0}
        # (a family that runs on the PyTorch operator set reads lengths on the host inside its forward: not capturable)
        self.use_graphs = bool(self.config.cuda_graphs and self.device.type == "cuda" and getattr(model, "supports_cuda_graphs", True))
        self.hybrid = mamba_shapes is not None
        # one-step lookahead of greedy graph decode: the step in flight whose sampled tokens the host has not read yet
        self._inflight: Optional[dict] = None
        # ("force" runs the same schedule without CUDA graphs: the host-side logic is then testable on a CPU)
        self.lookahead = bool(self.config.lookahead and (self.use_graphs or self.config.lookahead == "force"))
        if self.device.type == "cuda":
            e = ops.require_ext()
            e.init_scratch(self.device.index if self.device.index is not None else torch.cuda.current_device())

    def _auto_pages(self, layout) -> int:
        per = max(1, PagedKVCache.bytes_per_page(layout, self.config.kv.block_size, self.model.dtype))
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(free * self.config.kv_memory_fraction)
            # enough for max_seqs full contexts, never more than the budget
            want = self.config.max_seqs * ((self.cfg.max_position_embeddings + self.config.kv.block_size - 1) // self.config.kv.block_size) + 1
            return max(2, min(want, budget // per))
        return 2048

    # ------------------------------------------------------------------------------------------------ requests
    def add_request(self, prompt: list[int], params: Optional[GeneratorParameters] = None, on_token=None, guide=None,
                    stopper=None) -> Request:
        params = params or GeneratorParameters()
        params.validate()
        ctx = self.cfg.max_position_embeddings
        limit = min(params.ntokens or ctx, ctx)
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) >= limit:
            raise ValueError(f"prompt has {len(prompt)} tokens, which does not fit ntokens={limit}")
        if min(prompt) < 0 or max(prompt) >= self.cfg.vocab_size:
            raise ValueError(f"token ids must lie in [0, {self.cfg.vocab_size})")
        r = Request(self._next_id, [int(t) for t in prompt], params, on_token)
        self._next_id += 1
        r.sampling = SamplingState.create(params, self.special_ids)
        r.guide = guide
        r.stopper = stopper
        r.limit = limit
        r.t_submit = time.perf_counter()
        r.salt = compose_salt(params.cache_salt, params.lora_adapter or getattr(self.model, "active_lora", None),
                              self.model.tp.rank, self.model.tp.size)
        self.waiting.append(r)
        return r

    def abort(self, r: Request, reason: FinishReason = FinishReason.CANCELLED) -> None:
        r.cancelled = True
        if r.state == WAITING and r in self.waiting:
            self.waiting.remove(r)
            self._finish(r, reason)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    # ------------------------------------------------------------------------------------------------ scheduling
    def _admit(self, r: Request) -> bool:
        """Prefix lookup + page reservation for a waiting request."""
        if len(self.running) >= self.config.max_seqs:
            return False
        need_pages = (len(r.fill) + 1 + self.page_size - 1) // self.page_size
        # one page of headroom per running sequence: a request admitted into a nearly full pool would be preempted at once
        if not self.kv.can_allocate(need_pages + len(self.running)):
            return False
        if self.hybrid:
            if not self.kv.free_slots:
                return False
            r.state_slot = self.kv.alloc_state_slot()
        # Recurrent (conv / SSM) state is not idempotent: a snapshot taken after L tokens may only be resumed at token L. A hit
        # that covers the whole prompt would have to replay the last token on a state that already absorbed it, so hybrid
        # models only take checkpoints strictly shorter than the prompt and prefill the remainder from the restored state.
        hit = self.kv.prefix.lookup(r.salt, r.fill[:-1] if self.hybrid else r.fill)
        if hit is not None:
            r.pages = hit.pages
            r.prefix_hit = hit.length
            r.computed = hit.length
            if self.hybrid and hit.state is not None:
                self.kv.restore_state(r.state_slot, hit.state)
            if r.computed >= len(r.fill):
                r.computed = len(r.fill) - 1  # full hit: replay the last prompt token to get logits
        r.state = RUNNING
        self.running.append(r)
        return True

    def _finish(self, r: Request, reason: FinishReason) -> None:
        r.finish_reason = reason
        r.state = FINISHED
        r.t_done = time.perf_counter()
        if r in self.running:
            self.running.remove(r)
        self.kv.release_pages(r.pages)
        if r.state_slot >= 0:
            self.kv.free_state_slot(r.state_slot)
            r.state_slot = -1

    # ------------------------------------------------------------------------------------------------ memory pressure
    def _preempt(self, v: Request) -> None:
        """Take a running request out of the batch and give its pages back; it re-enters at the head of the waiting queue and
        rebuilds its cache by prefilling prompt + generated tokens (recompute; its own prompt is usually a prefix-cache hit).
        Sampling state, guide, stop detector and the tokens produced so far stay with the request, so its output is unchanged."""
        self.running.remove(v)
        self.kv.release_pages(v.pages)
        if v.state_slot >= 0:
            self.kv.free_state_slot(v.state_slot)
            v.state_slot = -1
        v.state, v.computed, v.state_snapshots = WAITING, 0, {}
        v.resumed = bool(v.output)
        v.fill = v.prompt + v.output[:-1] if v.output else v.prompt
        v.preemptions += 1
        self.metrics["preemptions"] = self.metrics.get("preemptions", 0) + 1
        self.waiting.insert(0, v)

    def _fail_oom(self, r: Request) -> None:
        """The oldest sequence cannot grow although nothing is left to preempt: the pool is too small for it. Only this
        request fails; :meth:`step` reports it with the other finished requests."""
        r.error = (f"KV cache is too small for this sequence ({r.total_len} tokens, {self.kv.num_pages - 1} pages of "
                   f"{self.page_size} tokens)")
        self._finish(r, FinishReason.ERROR)
        self._failed.append(r)

    def reset(self) -> None:
        """Drop every request and give all their pages and state slots back (after a fault in a step: the requests are failed
        by the caller, the engine must come back empty and leak nothing). Cached prefixes stay."""
        self._inflight = None
        for r in list(self.running) + list(self.waiting):
            r.pending = 0
            if r.state != FINISHED:
                if r in self.waiting:
                    self.waiting.remove(r)
                self._finish(r, FinishReason.ERROR)
        self.running.clear()
        self.waiting.clear()
        self._failed.clear()
        fused = getattr(getattr(self.model, "tp", None), "fused", None)
        if fused is not None and getattr(fused, "scatter", None) is not None:
            # its counters are cumulative across launches and ranks; after a failed step they may disagree, so prefill-size
            # projections go back to the GEMM + library all-reduce until the process group is rebuilt
            fused.scatter = None

    def _new_pages(self, r: Request, n_tokens: int) -> int:
        return max(0, (n_tokens + self.page_size - 1) // self.page_size - len(r.pages))

    def _reserve(self, r: Request, n_tokens: int) -> bool:
        """Pages for the first ``n_tokens`` positions of ``r``. Under pressure, requests admitted after ``r`` are preempted
        (youngest first); False when ``r`` has to wait for older requests to finish instead."""
        need = self._new_pages(r, n_tokens)
        while need > 0 and not self.kv.can_allocate(need):
            younger = self.running[self.running.index(r) + 1 :]
            victims = [v for v in younger if v.pending == 0]
            if not victims:
                if self.running[0] is r and not younger:
                    self._fail_oom(r)
                return False
            self._preempt(victims[-1])
        self.kv.ensure_pages(r.pages, n_tokens)
        return True

    def _make_room_for_decode(self, reqs: list[Request]) -> tuple:
        """Before a decode step: every sequence needs room for one more position (two with a token in flight). When the
        pool cannot supply that, the step in flight is settled and the youngest sequences are preempted until it can."""
        need = sum(self._new_pages(r, r.total_len + r.pending) for r in reqs)
        if need == 0 or self.kv.can_allocate(need):
            return reqs, []
        finished = self._drain()
        reqs = [r for r in reqs if r.state == RUNNING]
        while reqs and not self.kv.can_allocate(sum(self._new_pages(r, r.total_len) for r in reqs)):
            v = self.running[-1]  # youngest first; that may be a request whose prefill is waiting for pages
            if v is reqs[0]:
                self._fail_oom(v)
                reqs.remove(v)
                continue
            self._preempt(v)
            if v in reqs:
                reqs.remove(v)
        return reqs, finished

    def step(self) -> list[Request]:
        out = self._step()
        if self._failed:
            out = out + [r for r in self._failed if r not in out]
            self._failed.clear()
        return out

    def _step(self) -> list[Request]:
        """Run one engine step; returns the requests that finished in it. With lookahead decode the tokens of a decode step are
        read (and its finished requests reported) by the next call, while the device already runs the following step."""
        self.metrics["steps"] += 1
        finished: list[Request] = []
        for r in [x for x in self.running if x.cancelled]:
            if r.pending == 0:
                self._finish(r, FinishReason.CANCELLED)
                finished.append(r)
        if self.waiting and self._inflight is not None and len(self.running) < self.config.max_seqs:
            finished += self._drain()  # admissions and prefill work on settled request state
        # Admit only while this step's prefill budget has room: a request admitted later looks the prefix cache up later and
        # finds what the requests in front of it have stored by then (concurrent arrivals that share a prefix).
        backlog = sum(len(r.fill) - r.computed for r in self.running if r.computed < len(r.fill))
        while self.waiting and backlog < self.config.max_batch_tokens and self._admit(self.waiting[0]):
            r = self.waiting.pop(0)
            backlog += len(r.fill) - r.computed
        prefill = [r for r in self.running if r.computed < len(r.fill)]
        k = self.config.decode_interleave
        if prefill and k > 0 and self._prefill_streak >= k and any(r.computed >= len(r.fill) for r in self.running):
            prefill = []  # the running sequences get a decode step before the next prompt chunk
        self._prefill_streak = self._prefill_streak + 1 if prefill else 0
        if prefill:
            finished += self._drain()
            prefill = [r for r in prefill if r.state != FINISHED]
            out = self._prefill_step(prefill) if prefill else []
            if out is not None:
                return finished + out
            # every prefill of this step waits for pages that older, decoding requests hold: let those make progress
        ready = [r for r in self.running if r.computed >= len(r.fill)]
        if ready:
            return finished + self._decode_step(ready)
        if self._inflight is not None:
            return finished + self._drain()
        if self.waiting:
            raise MemoryError("waiting requests cannot be admitted: KV cache too small for the prompt")
        return finished

    # ------------------------------------------------------------------------------------------------ prefill
    def _prefill_step(self, reqs: list[Request]) -> Optional[list]:
        budget = self.config.max_batch_tokens
        seqs, chosen = [], []
        for r in reqs:
            if budget <= 0:
                break
            n = min(len(r.fill) - r.computed, budget)
            if self.hybrid:
                # recurrent state can only be snapshotted at chunk ends: stop chunks at the prefix-cache checkpoints
                for L in self.kv.settings.checkpoint_lengths(len(r.fill)):
                    if r.computed < L < r.computed + n:
                        n = L - r.computed
                        break
            if r.state != RUNNING or not self._reserve(r, r.computed + n):
                continue  # preempted by an older request of this step, or waiting for older requests to release pages
            seqs.append({"tokens": r.fill[r.computed : r.computed + n], "start": r.computed, "pages": r.pages,
                         "state_slot": max(r.state_slot, 0)})
            chosen.append((r, n))
            budget -= n
        if not seqs:
            return None
        batch = make_batch(seqs, self.page_size, self.device)
        logits = self.model.forward(batch, self.kv)
        self.metrics["prefill_steps"] += 1
        self.metrics["prefill_tokens"] += batch.num_tokens
        done_rows, done_reqs = [], []
        now = time.perf_counter()
        for i, (r, n) in enumerate(chosen):
            r.computed += n
            if r.computed < len(r.fill) and now - max(r.t_progress, r.t_submit) >= 3.0:
                # long prompts: a progress line every 3 s (the reference logs prefill progress the same way, AbstractModel.java:1126-1148)
                r.t_progress = now
                rate = (r.computed - r.prefix_hit) / max(now - r.t_submit, 1e-9)
                _log.info("prefill progress request=%d tokens=%d/%d rate=%.0f tok/s eta=%.1f s", r.rid, r.computed, len(r.fill), rate,
                          (len(r.fill) - r.computed) / max(rate, 1e-9))
            if self.hybrid and r.computed in self.kv.settings.checkpoint_lengths(len(r.fill)):
                r.state_snapshots[r.computed] = self.kv.snapshot_state(r.state_slot)
            if r.computed >= len(r.fill):
                self.kv.prefix.store(r.salt, r.fill, r.pages, r.state_snapshots if self.hybrid else None)
                if r.resumed:  # cache rebuilt after a preemption: the next token was sampled before, decoding just continues
                    r.resumed = False
                    continue
                done_rows.append(i)
                done_reqs.append(r)
        finished = []
        if done_reqs:
            sub = logits.index_select(0, torch.tensor(done_rows, device=logits.device)) if len(done_rows) != logits.shape[0] else logits
            finished = self._sample_and_advance(done_reqs, sub)
        return finished

    # ------------------------------------------------------------------------------------------------ decode
    def _decode_inputs(self, reqs: list[Request]):
        seqs = []
        for r in reqs:
            pos = r.total_len - 1 + r.pending  # position of the token being fed (the last sampled one)
            self.kv.ensure_pages(r.pages, pos + 1)
            seqs.append({"tokens": [r.output[-1] if r.output else 0], "start": pos, "pages": r.pages, "state_slot": max(r.state_slot, 0),
                         "rid": (r.rid, r.preemptions)})
        return seqs

    def _plain_greedy(self, reqs: list[Request]) -> bool:
        return all(r.guide is None and r.sampling.greedy and not r.params.logprobs for r in reqs)

    def _decode_step(self, reqs: list[Request]) -> list[Request]:
        reqs, early = self._make_room_for_decode(reqs)
        if early or not reqs:
            return early + (self._decode_step(reqs) if reqs else [])
        B = len(reqs)
        # (a request one token short of its context limit is settled synchronously: the surplus token of a lookahead step would
        # need a position and a page beyond the limit)
        if self.lookahead and B <= _BUCKETS[-1] and self._plain_greedy(reqs) and all(r.total_len + r.pending + 1 < r.limit for r in reqs):
            return self._lookahead_decode(reqs)
        finished = self._drain()
        reqs = [r for r in reqs if r.state != FINISHED]
        if not reqs:
            return finished
        B = len(reqs)
        seqs = self._decode_inputs(reqs)
        self.metrics["decode_steps"] += 1
        self.metrics["decode_tokens"] += B
        if self.use_graphs and B <= _BUCKETS[-1]:
            logits = self._graph_decode(seqs)[:B]
        else:
            batch = make_batch(seqs, self.page_size, self.device)
            batch.decode_splits = self._splits(B)
            logits = self.model.forward(batch, self.kv)
        return finished + self._sample_and_advance(reqs, logits)

    def _lookahead_decode(self, reqs: list[Request]) -> list[Request]:
        """Launch the decode step of ``reqs`` with the previous step's tokens still on the device, then settle the previous step
        on the host while this one runs. A request that turns out to have finished in the previous step has one surplus token
        computed, which is dropped; its pages are released only after this launch, so nothing reads them late."""
        prev = self._inflight
        B = len(reqs)
        dev_tokens = None
        if prev is not None:
            where = {id(r): i for i, r in enumerate(prev["reqs"])}
            if any(r.pending and id(r) not in where for r in reqs) or any(not r.pending for r in reqs):
                # the batch gained a member that is not part of the step in flight: settle first
                finished = self._drain()
                reqs = [r for r in reqs if r.state != FINISHED]
                return finished + (self._decode_step(reqs) if reqs else [])
            rows = [where[id(r)] for r in reqs]
            dev_tokens = prev["tokens"]
            if rows != list(range(len(prev["reqs"]))):
                dev_tokens = dev_tokens.index_select(0, torch.tensor(rows, device=dev_tokens.device))
        seqs = self._decode_inputs(reqs)
        self.metrics["decode_steps"] += 1
        self.metrics["decode_tokens"] += B
        if self.use_graphs:
            logits = self._graph_decode(seqs, dev_tokens)[:B]
        else:
            if dev_tokens is not None:
                for sq, t in zip(seqs, dev_tokens.tolist()):
                    sq["tokens"] = [int(t)]
            batch = make_batch(seqs, self.page_size, self.device)
            batch.decode_splits = self._splits(B)
            logits = self.model.forward(batch, self.kv)
        idx = self._greedy(logits)
        ev = None
        if self.device.type == "cuda":
            slot = self.metrics["decode_steps"] & 1
            if not hasattr(self, "_tok_host"):
                self._tok_host = [torch.zeros(_BUCKETS[-1], dtype=torch.int64).pin_memory() for _ in range(2)]
            host = self._tok_host[slot]
            host[:B].copy_(idx, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            host = idx.clone()
        for r in reqs:
            r.pending = 1
        self._inflight = {"reqs": list(reqs), "tokens": idx, "host": host, "event": ev}
        return self._settle(prev) if prev is not None else []

    def _settle(self, step: dict) -> list[Request]:
        """Read the sampled tokens of a launched step and run the per-request bookkeeping."""
        if step["event"] is not None:
            self._wait_event(step["event"])
        tokens = step["host"][: len(step["reqs"])].tolist()
        live, toks = [], []
        for r, t in zip(step["reqs"], tokens):
            if r.state != FINISHED:
                r.pending = 0
                live.append(r)
                toks.append(t)
        finished = self._advance(live, toks, [None] * len(live))
        if self._inflight is not None and self._inflight is not step:
            for r in live:  # still part of the step that is running now
                if r.state != FINISHED and any(r is x for x in self._inflight["reqs"]):
                    r.pending = 1
        return finished

    def _wait_event(self, ev) -> None:
        """Host-side watchdog: wait for a recorded event, but give up after ``device_timeout_s`` so that a device that stopped
        answering fails the requests in flight (the runner isolates the fault) instead of blocking the serving thread forever."""
        if ev.query():
            return
        t0 = time.perf_counter()
        pause = 20e-6
        while not ev.query():
            if time.perf_counter() - t0 > self.config.device_timeout_s:
                raise RuntimeError(f"device did not finish a decode step within {self.config.device_timeout_s:.0f} s")
            time.sleep(pause)
            pause = min(pause * 1.5, 2e-4)

    def _drain(self) -> list[Request]:
        step, self._inflight = self._inflight, None
        return self._settle(step) if step is not None else []

    def _splits(self, B: int) -> int:
        """Split-KV factor of decode attention: the smallest one that fills the resident CTA slots (two CTAs per SM) evenly."""
        ctas = max(1, B * self.model.n_kv)
        slots = 2 * 148
        best, best_eff = 1, 0.0
        for s in range(1, 33):
            n = ctas * s
            eff = n / (-(-n // slots) * slots)
            if eff > best_eff + 0.03:
                best, best_eff = s, eff
        return best

    def _graph_decode(self, seqs: list[dict], dev_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        B = len(seqs)
        bucket = next(b for b in _BUCKETS if b >= B)
        g = self._graphs.get(bucket)
        if g is None:
            g = self._capture(bucket)
        # stage inputs in pinned host buffers, one H2D copy per tensor
        # Two staging sets used in turn: the H2D copies below are asynchronous, and with lookahead decode the host stages step
        # N + 1 while the copies of step N may still be queued. A set is reused for step N + 2, which is staged only after the
        # event recorded behind step N has been waited for, i.e. after its copies have been read.
        ps = self.page_size
        slot = g["calls"] & 1
        g["calls"] += 1
        h = g["host"][slot]
        n = len(seqs)
        starts = [s["start"] for s in seqs]
        h["tok"][:n] = torch.tensor([s["tokens"][0] for s in seqs], dtype=torch.int32)
        h["pos"][:n] = torch.tensor(starts, dtype=torch.int32)
        h["slots"][:n] = torch.tensor([s["pages"][p // ps] * ps + p % ps for s, p in zip(seqs, starts)], dtype=torch.int64)
        h["ctx"][:n] = torch.tensor([p + 1 for p in starts], dtype=torch.int32)
        width = max(len(s["pages"]) for s in seqs)
        bt = h["bt"]
        owners = g["bt_owners"][slot]
        for i, s in enumerate(seqs):
            pg = s["pages"]
            key = (s.get("rid"), len(pg))  # between preemptions a request's page list only grows: same owner and length = same row
            if key[0] is not None and owners[i] == key:
                continue
            owners[i] = key
            row = s.get("bt_row")
            if row is not None:
                bt[i, : len(pg)] = row[: len(pg)]
            else:
                bt[i, : len(pg)] = torch.tensor(pg, dtype=torch.int32)
        for i in range(n, bucket):
            owners[i] = None
        if self.hybrid:
            h["st"][:n] = torch.tensor([s["state_slot"] for s in seqs], dtype=torch.int64)
        if n < bucket:
            h["tok"][n:] = 0
            h["pos"][n:] = 0
            h["ctx"][n:] = 1
            h["slots"][n:] = torch.arange(n, bucket, dtype=torch.int64) % ps  # padded rows write into the scratch page
            bt[n:, :1] = 0
        b: ForwardBatch = g["batch"]
        b.token_ids.copy_(h["tok"], non_blocking=True)
        if dev_tokens is not None:  # lookahead: the previous step's samples never left the device
            b.token_ids[:n].copy_(dev_tokens[:n])
        b.positions.copy_(h["pos"], non_blocking=True)
        b.slots.copy_(h["slots"], non_blocking=True)
        b.ctx_len.copy_(h["ctx"], non_blocking=True)
        b.block_tables[:, :width].copy_(bt[:, :width], non_blocking=True)
        if b.state_slots is not None:
            b.state_slots.copy_(h["st"], non_blocking=True)
        self.metrics["h2d_bytes"] = self.metrics.get("h2d_bytes", 0) + bucket * (4 + 4 + 8 + 4 + 4 * width)
        g["graph"].replay()
        self.metrics["graph_replays"] += 1
        self.metrics["kernel_launches"] += g["launches"]
        return g["logits"]

    def _capture(self, bucket: int) -> dict:
        dev = self.device
        batch = ForwardBatch(
            token_ids=torch.zeros(bucket, dtype=torch.int32, device=dev),
            positions=torch.zeros(bucket, dtype=torch.int32, device=dev),
            slots=torch.arange(bucket, dtype=torch.int64, device=dev) % self.page_size,
            q_start=torch.arange(bucket, dtype=torch.int32, device=dev),
            q_len=torch.ones(bucket, dtype=torch.int32, device=dev),
            ctx_len=torch.ones(bucket, dtype=torch.int32, device=dev),
            block_tables=torch.zeros(bucket, self.max_pages_per_seq, dtype=torch.int32, device=dev),
            is_decode=True,
            logits_rows=torch.arange(bucket, dtype=torch.int64, device=dev),
            decode_splits=self._splits(bucket),
            state_slots=torch.zeros(bucket, dtype=torch.int64, device=dev) if self.hybrid else None,
        )
        # warm up outside capture (lazy handles, function attributes, scratch), then capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(batch, self.kv)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        n0 = ops.LAUNCHES[0]
        with torch.cuda.graph(graph):
            logits = self.model.forward(batch, self.kv)
        launches = ops.LAUNCHES[0] - n0
        pin = dev.type == "cuda"
        host = [{
            "tok": torch.zeros(bucket, dtype=torch.int32, pin_memory=pin),
            "pos": torch.zeros(bucket, dtype=torch.int32, pin_memory=pin),
            "slots": torch.zeros(bucket, dtype=torch.int64, pin_memory=pin),
            "ctx": torch.ones(bucket, dtype=torch.int32, pin_memory=pin),
            "bt": torch.zeros(bucket, self.max_pages_per_seq, dtype=torch.int32, pin_memory=pin),
            "st": torch.zeros(bucket, dtype=torch.int64, pin_memory=pin),
        } for _ in range(2)]
        g = {"graph": graph, "batch": batch, "logits": logits, "host": host, "launches": launches, "calls": 0,
             "bt_owners": [[None] * bucket, [None] * bucket]}
        self._graphs[bucket] = g
        return g

    # ------------------------------------------------------------------------------------------------ sampling / stops
    def _sample_and_advance(self, reqs: list[Request], logits: torch.Tensor) -> list[Request]:
        cfg = self.cfg
        mask = None
        if any(r.guide is not None for r in reqs):
            words = (cfg.vocab_size + 31) // 32
            dev = logits.device
            if dev.type == "cuda":
                # masks live on the device per automaton state (uploaded once); the step only gathers rows
                mask = torch.full((len(reqs), words), -1, dtype=torch.int32, device=dev)
                idx, rows = [], []
                for i, r in enumerate(reqs):
                    if r.guide is not None:
                        on = getattr(r.guide, "allowed_mask_on", None)
                        rows.append(on(dev) if on is not None else r.guide.allowed_mask().to(dev))
                        idx.append(i)
                mask[torch.tensor(idx, device=dev)] = torch.stack(rows)
            else:
                m = torch.full((len(reqs), words), -1, dtype=torch.int32)
                for i, r in enumerate(reqs):
                    if r.guide is not None:
                        m[i] = r.guide.allowed_mask()
                mask = m
        inv_scale = 1.0 / cfg.logits_scaling if cfg.logits_scaling not in (0.0, 1.0) else 1.0
        all_greedy_plain = mask is None and all(r.sampling.greedy and not r.params.logprobs for r in reqs)
        if all_greedy_plain:
            tokens = self._greedy(logits).tolist()  # softcap and positive scaling keep the argmax
            lps = [None] * len(reqs)
        else:
            logits = self._full(logits)
            if mask is not None or cfg.final_softcap > 0 or inv_scale != 1.0:
                logits = ops.logits_post(logits if not self.use_graphs else logits.clone(), mask, cfg.final_softcap, inv_scale)
            tokens, lps = self.sampler.sample(logits, [r.sampling for r in reqs])
        return self._advance(reqs, tokens, lps)

    def _greedy(self, logits: torch.Tensor) -> torch.Tensor:
        fn = getattr(self.model, "greedy_tokens", None)
        return fn(logits) if fn is not None else ops.argmax(logits)[0]

    def _full(self, logits: torch.Tensor) -> torch.Tensor:
        fn = getattr(self.model, "full_logits", None)
        return fn(logits) if fn is not None else logits

    def _advance(self, reqs: list[Request], tokens: list, lps: list) -> list[Request]:
        now = time.perf_counter()
        finished = []
        for r, tok, lp in zip(reqs, tokens, lps):
            if not r.output:
                r.t_first = now
            r.output.append(int(tok))
            if lp is not None:
                r.logprobs.append(lp)
            if r.guide is not None:
                r.guide.accept(int(tok))
            reason = self._stop_reason(r, int(tok))
            if r.on_token is not None:
                try:
                    r.on_token(int(tok), r)
                except Exception as e:  # a failing callback cancels only its own request
                    r.error = repr(e)
                    reason = reason or FinishReason.ERROR
            if reason is None and r.stopper is not None:
                reason = r.stopper.check(r)
            if reason is None and int(tok) in self.eos_ids:
                reason = FinishReason.STOP_TOKEN
            if reason is None and r.total_len >= r.limit:
                reason = FinishReason.MAX_TOKENS
            if reason is None and r.cancelled:
                reason = FinishReason.CANCELLED
            if reason is not None:
                self._finish(r, reason)
                finished.append(r)
        return finished

    def _stop_reason(self, r: Request, tok: int) -> Optional[FinishReason]:
        if r.params.max_tokens is not None and len(r.output) >= r.params.max_tokens:
            return FinishReason.MAX_TOKENS
        if r.guide is not None and getattr(r.guide, "is_complete", lambda: False)():
            return FinishReason.GUIDED_COMPLETE
        return None

    # ------------------------------------------------------------------------------------------------ conveniences
    def run(self, reqs: Optional[list[Request]] = None) -> None:
        while self.has_work() and (reqs is None or any(r.state != FINISHED for r in reqs)):
            self.step()

    def generate(self, prompt: list[int], params: Optional[GeneratorParameters] = None, on_token=None, guide=None,
                 stopper=None) -> Response:
        r = self.add_request(prompt, params, on_token, guide, stopper)
        self.run([r])
        if self.device.type == "cuda":
            ops.check_status(self.device.index)
        if r.finish_reason == FinishReason.ERROR and r.error and r.error.startswith("KV cache is too small"):
            raise MemoryError(r.error)
        return r.response()

    def generate_batch(self, prompts: list[list[int]], params: Optional[GeneratorParameters] = None) -> list[Response]:
        import copy

        rs = [self.add_request(p, copy.deepcopy(params) if params else None) for p in prompts]
        self.run(rs)
        if self.device.type == "cuda":
            ops.check_status(self.device.index)
        return [r.response() for r in rs]
