"""One-node rank supervisor: starts one process per GPU, watches them, and restarts the whole group when a rank dies or hangs.

    python -m deliverance_b200.parallel.cluster --nproc 8 [--max-restarts 3] [--hang-timeout 60] -- \
        python -m deliverance_b200.server --model /models/Qwen3-4B-JQ4 --port 8080

What it replaces. The reference runs tensor-parallel roles as separate JVMs started by a launcher
(core/.../benchmark/TpLocalCluster.java:246-274), finds them through UDP gossip, elects a leader that publishes a rank
assignment, and every worker runs a reconcile loop that stops and restarts its local ranks when the assignment changes
(core/.../model/tensorparallel/GossipParallelMembership.java:197-218, 368-416). On one NVSwitch node the membership is static
(``RANK`` / ``WORLD_SIZE`` from the environment), so what is left of that machinery is: launch the ranks, notice a failed or
silent rank, and bring the group back. A collective group cannot continue with a missing member (peer-memory slabs and NCCL
communicators are created for a fixed size), so recovery is always a restart of ALL ranks with a fresh rendezvous port.

Failure detection is host-side only:
  * a child that exits (any code) while the group is meant to run is a failure; ``--exit-ok`` lets a group end normally when
    every rank exits 0;
  * ranks may publish liveness by touching ``$DLV_HEARTBEAT_DIR/rank<R>`` (``beat()`` below; the lockstep serving loop does it
    once per step): a rank whose file is older than ``hang_timeout`` seconds is treated as hung.
Children are stopped by their exact process ids (SIGTERM, then SIGKILL after a grace period), never by name.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import socket
import subprocess
import sys
import tempfile
import threading
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

_BEAT_PATH: Optional[str] = None
_BEAT_LAST = 0.0


def beat(min_interval: float = 0.2) -> None:
    """Called by a rank to say it is alive (cheap: at most one ``utime`` per ``min_interval`` seconds; no-op when the
    process was not started by the supervisor)."""
    global _BEAT_PATH, _BEAT_LAST
    if _BEAT_PATH is None:
        d = os.environ.get("DLV_HEARTBEAT_DIR")
        _BEAT_PATH = os.path.join(d, f"rank{os.environ.get('RANK', '0')}") if d else ""
    if not _BEAT_PATH:
        return
    now = time.monotonic()
    if now - _BEAT_LAST < min_interval:
        return
    _BEAT_LAST = now
    with open(_BEAT_PATH, "a"):
        os.utime(_BEAT_PATH, None)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@dataclass
class ClusterStatus:
    generation: int = 0  # how many times the group has been (re)started
    restarts: int = 0
    state: str = "idle"  # idle | running | restarting | finished | failed
    last_failure: str = ""
    pids: list = field(default_factory=list)
    failures: list = field(default_factory=list)

    def to_json(self) -> dict:
        return {"generation": self.generation, "restarts": self.restarts, "state": self.state, "last_failure": self.last_failure,
                "pids": list(self.pids), "failures": list(self.failures)}


class LocalCluster:
    def __init__(self, cmd: Sequence[str], nproc: int, max_restarts: int = 3, hang_timeout: float = 0.0, exit_ok: bool = True,
                 grace: float = 5.0, poll: float = 0.1, env: Optional[dict] = None, status_file: Optional[str] = None,
                 start_timeout: float = 0.0):
        self.cmd, self.nproc = list(cmd), nproc
        self.max_restarts, self.hang_timeout, self.exit_ok = max_restarts, hang_timeout, exit_ok
        self.grace, self.poll = grace, poll
        self.env = dict(env if env is not None else os.environ)
        self.status_file = status_file
        # a rank must publish its first heartbeat within this many seconds; loading a model takes far longer than a step
        self.start_timeout = start_timeout or (max(10 * hang_timeout, 600.0) if hang_timeout > 0 else 0.0)
        self.status = ClusterStatus()
        self.procs: list[subprocess.Popen] = []
        self.hb_dir = tempfile.mkdtemp(prefix="dlv_hb_")
        self._stop = threading.Event()

    # ------------------------------------------------------------------------------------------------ group lifecycle
    def _spawn(self) -> None:
        port = _free_port()
        for r in range(self.nproc):
            p = os.path.join(self.hb_dir, f"rank{r}")
            if os.path.exists(p):
                os.unlink(p)
        self.procs = []
        for r in range(self.nproc):
            e = dict(self.env)
            e.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(self.nproc), LOCAL_WORLD_SIZE=str(self.nproc), MASTER_ADDR="127.0.0.1",
                     MASTER_PORT=str(port), DLV_HEARTBEAT_DIR=self.hb_dir, DLV_RESTART_COUNT=str(self.status.restarts))
            if self.status_file:
                e["DLV_CLUSTER_STATUS_FILE"] = self.status_file
            self.procs.append(subprocess.Popen(self.cmd, env=e, start_new_session=True))
        self.status.generation += 1
        self.status.state = "running"
        self.status.pids = [p.pid for p in self.procs]
        self._t_spawn = time.monotonic()
        self._publish()

    def _stop_group(self) -> None:
        """Stop every child that is still running: SIGTERM to its own process group, SIGKILL after the grace period."""
        live = [p for p in self.procs if p.poll() is None]
        for p in live:
            try:
                os.killpg(p.pid, signal.SIGTERM)  # the child leads its own session (start_new_session), so pgid == pid
            except ProcessLookupError:
                pass
        t_end = time.monotonic() + self.grace
        for p in live:
            try:
                p.wait(max(0.0, t_end - time.monotonic()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                p.wait()

    def _check(self) -> Optional[str]:
        """None while healthy; "done" when every rank exited 0 (and that is allowed); otherwise a failure description."""
        codes = [p.poll() for p in self.procs]
        if all(c is not None for c in codes):
            if self.exit_ok and all(c == 0 for c in codes):
                return "done"
            return "all ranks exited: codes " + ",".join(str(c) for c in codes)
        for r, c in enumerate(codes):
            if c is not None and not (self.exit_ok and c == 0):
                return f"rank {r} (pid {self.procs[r].pid}) exited with code {c}"
        if self.hang_timeout > 0:
            now_wall, since = time.time(), time.monotonic() - self._t_spawn
            for r, c in enumerate(codes):
                if c is not None:
                    continue
                p = os.path.join(self.hb_dir, f"rank{r}")
                if os.path.exists(p):
                    age = now_wall - os.path.getmtime(p)
                    if age > self.hang_timeout:
                        return f"rank {r} (pid {self.procs[r].pid}) silent for {age:.1f} s"
                elif self.start_timeout > 0 and since > self.start_timeout:
                    return f"rank {r} (pid {self.procs[r].pid}) published no heartbeat within {since:.1f} s of start"
        return None

    def _publish(self) -> None:
        if self.status_file:
            tmp = self.status_file + ".tmp"
            with open(tmp, "w") as f:
                json.dump(self.status.to_json(), f)
            os.replace(tmp, self.status_file)

    def run(self) -> int:
        """Blocks until the group finished (0), was stopped (0) or failed more often than ``max_restarts`` allows (1)."""
        self._spawn()
        try:
            while not self._stop.is_set():
                time.sleep(self.poll)
                verdict = self._check()
                if verdict is None:
                    continue
                if verdict == "done":
                    self.status.state = "finished"
                    self._publish()
                    return 0
                self.status.last_failure = verdict
                self.status.failures.append({"generation": self.status.generation, "what": verdict, "t": time.time()})
                print(f"[cluster] {verdict}; stopping the group", file=sys.stderr, flush=True)
                self.status.state = "restarting"
                self._publish()
                self._stop_group()
                if self.status.restarts >= self.max_restarts:
                    self.status.state = "failed"
                    self._publish()
                    print(f"[cluster] giving up after {self.status.restarts} restarts", file=sys.stderr, flush=True)
                    return 1
                self.status.restarts += 1
                self._spawn()
            return 0
        finally:
            self._stop_group()
            if self.status.state == "running":
                self.status.state = "idle"
            self._publish()

    def stop(self) -> None:
        self._stop.set()


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--" not in argv:
        raise SystemExit("usage: python -m deliverance_b200.parallel.cluster --nproc N [options] -- <command of one rank>")
    i = argv.index("--")
    ap = argparse.ArgumentParser(prog="deliverance_b200.parallel.cluster")
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--hang-timeout", type=float, default=0.0, help="seconds without a heartbeat before a rank counts as hung (0: off)")
    ap.add_argument("--start-timeout", type=float, default=0.0, help="seconds a rank may take to publish its first heartbeat (model load)")
    ap.add_argument("--no-exit-ok", action="store_true", help="treat any exit of a rank as a failure (servers)")
    ap.add_argument("--status-file", default=None, help="JSON status written on every change (served by GET /tp/status)")
    a = ap.parse_args(argv[:i])
    c = LocalCluster(argv[i + 1 :], a.nproc, a.max_restarts, a.hang_timeout, not a.no_exit_ok, status_file=a.status_file,
                     start_timeout=a.start_timeout)
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: c.stop())
    return c.run()


if __name__ == "__main__":
    raise SystemExit(main())
