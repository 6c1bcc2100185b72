"""Engine loop thread: the bridge between concurrent callers (HTTP handlers) and the single-threaded engine.

The reference starts one ``model.generate`` per HTTP request on a common pool with no queue or admission control
(web/.../ChatCompletionController.java:373-383). Here every caller submits to one runner; the runner thread owns the
engine, admits requests between steps (continuous batching) and delivers token events through thread-safe callbacks.
Cancellation (client disconnect) marks the request and is honoured before the next step.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Callable, Optional

from ..api import CausalLanguageModel, Generation
from ..params import GeneratorParameters, Response


class Submission:
    def __init__(self, prompt, params, on_event, on_done, session):
        self.prompt, self.params, self.on_event, self.on_done, self.session = prompt, params, on_event, on_done, session
        self.generation: Optional[Generation] = None
        self.cancelled = False
        self.done = threading.Event()
        self.response: Optional[Response] = None
        self.error: Optional[BaseException] = None

    def cancel(self) -> None:
        self.cancelled = True

    def wait(self, timeout: Optional[float] = None) -> Response:
        if not self.done.wait(timeout):
            raise TimeoutError("generation did not finish in time")
        if self.error is not None:
            raise self.error
        return self.response


class EngineRunner:
    def __init__(self, clm: CausalLanguageModel, idle_sleep: float = 0.002):
        self.clm = clm
        self.inbox: "queue.Queue[Submission]" = queue.Queue()
        self.active: list[Submission] = []
        self.idle_sleep = idle_sleep
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._loop, name="deliverance-engine", daemon=True)
        self.stats = {"submitted": 0, "finished": 0, "errors": 0, "cancelled": 0}
        self.thread.start()

    def submit(self, prompt, params: Optional[GeneratorParameters] = None, on_event: Optional[Callable] = None,
               on_done: Optional[Callable] = None, session: Optional[str] = None) -> Submission:
        s = Submission(prompt, params or GeneratorParameters(), on_event, on_done, session)
        self.stats["submitted"] += 1
        self.inbox.put(s)
        return s

    def generate(self, prompt, params=None, on_event=None, session=None, timeout: Optional[float] = None) -> Response:
        return self.submit(prompt, params, on_event, None, session).wait(timeout)

    def _finish(self, s: Submission, error: Optional[BaseException] = None) -> None:
        if error is not None:
            s.error = error
            self.stats["errors"] += 1
        else:
            req = s.generation.request
            if req.finish_reason is not None and req.finish_reason.name == "ERROR" and req.error:
                s.error = RuntimeError(req.error)  # failed inside the engine (KV pool too small for it, failing callback)
                self.stats["errors"] += 1
            else:
                s.response = s.generation.finish()
                self.stats["finished"] += 1
        if s in self.active:
            self.active.remove(s)
        s.done.set()
        if s.on_done is not None:
            try:
                s.on_done(s)
            except Exception:  # noqa: BLE001 - a failing completion hook must not stop the loop
                pass

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                self._serve()
            except Exception as e:  # noqa: BLE001 - a bug in the bookkeeping must not leave callers waiting for a dead thread
                for s in list(self.active):
                    self._finish(s, e)
                try:
                    self.clm.engine.reset()
                except Exception:  # noqa: BLE001
                    pass

    def _serve(self) -> None:
        eng = self.clm.engine
        while not self._stop.is_set():
            try:
                while True:
                    s = self.inbox.get_nowait()
                    if s.cancelled:
                        self.stats["cancelled"] += 1
                        self._finish(s, RuntimeError("cancelled before start"))
                        continue
                    try:
                        s.generation = self.clm.submit(s.prompt, s.params, s.on_event, s.session)
                        self.active.append(s)
                    except Exception as e:  # noqa: BLE001 - bad request: report to the caller, keep serving
                        self._finish(s, e)
            except queue.Empty:
                pass
            for s in list(self.active):
                if s.cancelled and s.generation.request.state != "finished":
                    eng.abort(s.generation.request)
                    self.stats["cancelled"] += 1
            if not eng.has_work():
                for s in list(self.active):
                    if s.generation.request.state == "finished":
                        self._finish(s)
                time.sleep(self.idle_sleep)
                continue
            try:
                eng.step()
            except Exception as e:  # noqa: BLE001 - an engine fault fails the in-flight requests, not the server
                for s in list(self.active):
                    self._finish(s, e)
                try:
                    eng.reset()  # every request is dropped and its pages and state slots go back to the pool
                except Exception:  # noqa: BLE001 - bookkeeping damaged by the fault: start from empty queues at least
                    eng.running.clear()
                    eng.waiting.clear()
                continue
            for s in list(self.active):
                if s.generation.request.state == "finished":
                    self._finish(s)

    def _drain_on_stop(self) -> None:
        """The loop has ended: nobody will step the engine again, so callers still waiting are answered with an error instead of
        running into their time-outs, and the engine gives its pages back."""
        pending = list(self.active)
        try:
            while True:
                pending.append(self.inbox.get_nowait())
        except queue.Empty:
            pass
        for s in pending:
            if not s.done.is_set():
                self._finish(s, RuntimeError("server is shutting down"))
        try:
            self.clm.engine.reset()
        except Exception:  # noqa: BLE001
            pass

    def close(self) -> None:
        self._stop.set()
        self.thread.join(timeout=5)
        if not self.thread.is_alive():
            self._drain_on_stop()
