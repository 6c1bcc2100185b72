"""Stage profiler: named timers and counters around the inference stages, printed as ``[profile] name count total_ms mean_us``.

Same stage names and report format as the reference's ``InferenceProfiler`` (core/.../model/InferenceProfiler.java:24-161:
``generation.prefill/decode``, ``causalselfattention.{qkv_projection,rope,score_value,output_projection,all_reduce}``,
``mlpblock.*``, ``sampler.*``, ``guided.*``, ``kvbuffercache.prefix.*``) but timed on the device: each stage is bracketed by
CUDA events on the current stream and resolved at ``summary()`` (one synchronize), so the timers do not serialise the
stream. Path counters (``sampler.output_weight_Q4`` ...) record which kernel variant ran. Enabled with
``DELIVERANCE_PROFILE_STAGES=1`` or ``--profile-stages``; eager mode only (a captured CUDA graph replays without Python).
With ``DELIVERANCE_NVTX=1`` every stage also opens an NVTX range of the same name, so a timeline profiler shows the stages.
"""
from __future__ import annotations

import os
import time
from collections import defaultdict
from contextlib import contextmanager

import torch


class InferenceProfiler:
    def __init__(self, device=None, enabled: bool = True):
        self.enabled = enabled
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self._pending: dict[str, list] = defaultdict(list)
        self._totals: dict[str, float] = defaultdict(float)  # ms
        self._counts: dict[str, int] = defaultdict(int)
        self.counters: dict[str, int] = defaultdict(int)
        self.nvtx = self.cuda and bool(os.environ.get("DELIVERANCE_NVTX"))

    @staticmethod
    def from_env(device=None) -> "InferenceProfiler | None":
        return InferenceProfiler(device) if os.environ.get("DELIVERANCE_PROFILE_STAGES") else None

    @contextmanager
    def stage(self, name: str):
        if not self.enabled:
            yield
            return
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if self.nvtx:
                torch.cuda.nvtx.range_push(name)
            a.record()
            try:
                yield
            finally:
                b.record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self._pending[name].append((a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._totals[name] += (time.perf_counter() - t0) * 1e3
                self._counts[name] += 1

    def count(self, name: str, n: int = 1) -> None:
        if self.enabled:
            self.counters[name] += n

    def _resolve(self) -> None:
        if not self._pending:
            return
        torch.cuda.synchronize(self.device)
        for name, evs in self._pending.items():
            for a, b in evs:
                self._totals[name] += a.elapsed_time(b)
                self._counts[name] += 1
        self._pending.clear()

    def reset(self) -> None:
        self._resolve()
        self._totals.clear()
        self._counts.clear()
        self.counters.clear()

    def totals(self) -> dict[str, tuple[int, float]]:
        self._resolve()
        return {k: (self._counts[k], self._totals[k]) for k in self._totals}

    def summary(self) -> str:
        rows = sorted(self.totals().items(), key=lambda kv: -kv[1][1])
        lines = [f"[profile] {name} count={c} total_ms={ms:.3f} mean_us={ms * 1e3 / max(1, c):.2f}" for name, (c, ms) in rows]
        lines += [f"[profile-counter] {k} count={v}" for k, v in sorted(self.counters.items())]
        return "\n".join(lines)

    def print_summary(self) -> None:
        print(self.summary())
