"""Tensor-parallel serving in lockstep: rank 0 owns the HTTP front end, every rank owns one shard of the model.

The reference keeps tensor-parallel workers in step by having the coordinator call every rank's ``/forward`` or
``/batchForward`` endpoint for each token (core/.../model/tensorparallel/TensorParallelGenerationGroup.java:216-235; its
workers never see a request). Here all
ranks run the same continuous-batching engine. What must be identical on every rank is the sequence of engine
operations: which requests are admitted or cancelled before which step. Rank 0 therefore publishes one small command per
loop iteration through a control group (gloo or thread ranks, never the NCCL stream): the token ids and parameters of new
requests, the sessions to cancel, and whether to stop. Followers apply the command and step. Sampling needs no extra
traffic: logits are bit-identical on all ranks after the rank-ordered all-reduce, and every request carries its seed.

Failure model: a follower that hears nothing for ``timeout`` seconds (rank 0 sends an idle heartbeat at least every
``heartbeat`` seconds) leaves its loop with an error; rank 0 learns of a dead follower from the control group's own timeout
on the next broadcast and fails the in-flight requests instead of hanging the server.
"""
from __future__ import annotations

import copy
import queue
import time
from typing import Optional

from ..api import CausalLanguageModel
from ..parallel.context import Collectives
from ..parallel.cluster import beat
from ..prompt.chat import PromptContext
from .runner import EngineRunner, Submission


def _command(new=(), cancel=(), stop=False, reset=False) -> dict:
    return {"new": list(new), "cancel": list(cancel), "stop": bool(stop), "reset": bool(reset)}


class LockstepRunner(EngineRunner):
    """Rank-0 runner: like :class:`EngineRunner`, but every admission / cancellation is first broadcast to the followers."""

    def __init__(self, clm: CausalLanguageModel, control: Collectives, idle_sleep: float = 0.002, heartbeat: float = 0.5):
        self.control = control
        self.heartbeat = heartbeat
        self._announced_cancel: set = set()
        super().__init__(clm, idle_sleep)

    def _loop(self) -> None:
        eng = self.clm.engine
        last_sent = 0.0
        while True:
            beat()  # liveness for the rank supervisor (parallel/cluster.py); no-op when not supervised
            stop = self._stop.is_set()
            fresh: list[Submission] = []
            try:
                while True:
                    s = self.inbox.get_nowait()
                    if s.cancelled:
                        self.stats["cancelled"] += 1
                        self._finish(s, RuntimeError("cancelled before start"))
                    else:
                        fresh.append(s)
            except queue.Empty:
                pass
            # A request is submitted to rank 0's engine BEFORE it is announced: only requests that the engine and the guide
            # compiler accepted (prompt length, parameters, guided regex / schema, adapter id) reach the followers, so a malformed
            # client request is answered with an error here and never costs a follower. No step runs between this point and the
            # followers' own submit, so every rank still sees the same sequence of engine operations.
            new = []
            for s in fresh:
                try:
                    has_tools = isinstance(s.prompt, PromptContext) and s.prompt.has_tools
                    text = s.prompt.prompt if isinstance(s.prompt, PromptContext) else s.prompt
                    ids = self.clm.encode_prompt(text) if isinstance(text, str) else [int(t) for t in text]
                    s.session = s.session or f"s{self.stats['submitted']}-{id(s):x}"
                    announced = copy.deepcopy(s.params)
                    s.generation = self.clm.submit(PromptIds(ids, has_tools), s.params, s.on_event, s.session)
                    self.active.append(s)
                    new.append((ids, announced, has_tools, s.session))
                except Exception as e:  # noqa: BLE001 - bad request: report, keep serving
                    self._finish(s, e)
            cancel = [s.session for s in self.active if s.cancelled and s.session not in self._announced_cancel
                      and s.generation.request.state != "finished"]
            busy = eng.has_work() or new or cancel or stop or getattr(self, "_reset_followers", False)
            if not busy and time.monotonic() - last_sent < self.heartbeat:
                for s in list(self.active):
                    if s.generation.request.state == "finished":
                        self._finish(s)
                time.sleep(self.idle_sleep)
                continue
            try:
                self.control.broadcast_object(_command(new, cancel, stop, getattr(self, "_reset_followers", False)), 0)
                self._reset_followers = False
                last_sent = time.monotonic()
            except Exception as e:  # noqa: BLE001 - a follower is gone: fail what is in flight
                for s in list(self.active):
                    self._finish(s, RuntimeError(f"tensor-parallel control group failed: {e}"))
                return
            if stop:
                return
            for s in list(self.active):
                if s.session in cancel:
                    self._announced_cancel.add(s.session)
                    eng.abort(s.generation.request)
                    self.stats["cancelled"] += 1
            if eng.has_work():
                try:
                    eng.step()
                except Exception as e:  # noqa: BLE001
                    for s in list(self.active):
                        self._finish(s, e)
                    try:
                        eng.reset()
                    except Exception:  # noqa: BLE001
                        eng.running.clear()
                        eng.waiting.clear()
                    self._reset_followers = True  # the other ranks drop their copies of the failed requests with the next command
                    continue
            for s in list(self.active):
                if s.generation.request.state == "finished":
                    self._announced_cancel.discard(s.session)
                    self._finish(s)

    def close(self) -> None:
        self._stop.set()
        self.thread.join(timeout=10)
        if not self.thread.is_alive():
            self._drain_on_stop()


class PromptIds(list):
    """Token ids that remember whether the request carried tools (tool-call stop handling depends on it)."""

    def __init__(self, ids, has_tools: bool = False):
        super().__init__(ids)
        self.has_tools = has_tools


def follower_loop(clm: CausalLanguageModel, control: Collectives, max_idle: Optional[float] = None) -> int:
    """Ranks > 0: apply rank 0's commands and step the engine until told to stop. Returns the number of steps run."""
    eng = clm.engine
    live: dict = {}
    steps = 0
    last = time.monotonic()
    while True:
        beat()
        cmd = control.broadcast_object(None, 0)
        if cmd is None:
            raise RuntimeError("control group delivered no command (coordinator gone?)")
        if cmd["new"] or cmd["cancel"] or eng.has_work():
            last = time.monotonic()
        elif max_idle is not None and time.monotonic() - last > max_idle:
            raise TimeoutError("no work from the coordinator")
        if cmd.get("reset"):  # rank 0 failed a step and dropped every request: drop them here too, before the new ones
            eng.reset()
            live.clear()
        if cmd["stop"]:
            return steps
        for ids, params, has_tools, session in cmd["new"]:
            try:
                live[session] = clm.submit(PromptIds(ids, has_tools), params, None, session)
            except Exception:  # noqa: BLE001 - rank 0 only announces what its own engine accepted; a rejection here must not end the rank
                live.pop(session, None)
        for session in cmd["cancel"]:
            g = live.get(session)
            if g is not None and g.request.state != "finished":
                eng.abort(g.request)
        if eng.has_work():
            eng.step()
            steps += 1
        for k in [k for k, g in live.items() if g.request.state == "finished"]:
            del live[k]
