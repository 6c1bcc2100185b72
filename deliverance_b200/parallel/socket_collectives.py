"""All-reduce-sum over TCP through a leader-hosted server: the CPU / multi-host fallback transport.

Protocol of the reference's Netty transport (core/.../tensorparallel/transport/NettyTensorParallelCollectives.java:37-186,
NettyTensorParallelCollectiveServer.java:38-290, HttpTensorParallelCollectiveServer.java:140-196): one persistent connection
per rank, frames ``u32 length | u8 type | body``; an all-reduce request carries ``u32 headerLen | JSON {key, rank, size} |
DTEN tensor``; the server collects ``size`` contributions per wire key ``session:<id>:<seq>:<key>``, adds them in rank order
and answers every caller with the sum; a contribution that waits longer than the timeout fails with the key and the ranks
that did arrive. On a B200 node this path is never used for tensors (NVLink peer memory is); it serves CPU ranks and tests.
"""
from __future__ import annotations

import json
import socket
import struct
import threading
import time

import torch

from . import dten
from .context import Collectives

MSG_ALLREDUCE, MSG_RESULT, MSG_ERROR = 1, 2, 3
MAX_FRAME = 256 << 20


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    chunks, got = [], 0
    while got < n:
        b = sock.recv(min(1 << 20, n - got))
        if not b:
            raise ConnectionError("peer closed the connection")
        chunks.append(b)
        got += len(b)
    return b"".join(chunks)


def _send_frame(sock: socket.socket, mtype: int, body: bytes) -> None:
    if len(body) + 1 > MAX_FRAME:
        raise ValueError("frame exceeds 256 MiB")
    sock.sendall(struct.pack("<IB", len(body) + 1, mtype) + body)


def _recv_frame(sock: socket.socket) -> tuple[int, bytes]:
    (n,) = struct.unpack("<I", _recv_exact(sock, 4))
    if n < 1 or n > MAX_FRAME:
        raise ValueError(f"bad frame length {n}")
    data = _recv_exact(sock, n)
    return data[0], data[1:]


class CollectiveServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, timeout: float = 30.0):
        self.timeout = timeout
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((host, port))
        self._sock.listen(64)
        self.address = self._sock.getsockname()
        self._cv = threading.Condition()
        self._groups: dict[str, dict] = {}
        self._stop = False
        self.stats = {"requests": 0, "timeouts": 0}
        threading.Thread(target=self._accept, daemon=True, name="dlv-collective-accept").start()

    def _accept(self) -> None:
        while not self._stop:
            try:
                c, _ = self._sock.accept()
            except OSError:
                return
            c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            threading.Thread(target=self._serve, args=(c,), daemon=True).start()

    def _serve(self, c: socket.socket) -> None:
        try:
            while True:
                mtype, body = _recv_frame(c)
                if mtype != MSG_ALLREDUCE:
                    _send_frame(c, MSG_ERROR, b"unknown message type")
                    continue
                (hlen,) = struct.unpack_from("<I", body, 0)
                hdr = json.loads(body[4 : 4 + hlen])
                t = dten.decode(body[4 + hlen :])
                try:
                    out = self._reduce(hdr["key"], int(hdr["rank"]), int(hdr["size"]), t)
                    _send_frame(c, MSG_RESULT, dten.encode(out))
                except TimeoutError as e:
                    _send_frame(c, MSG_ERROR, str(e).encode())
        except (ConnectionError, OSError, ValueError):
            pass
        finally:
            c.close()

    def _reduce(self, key: str, rank: int, size: int, t: torch.Tensor) -> torch.Tensor:
        self.stats["requests"] += 1
        with self._cv:
            g = self._groups.setdefault(key, {"vals": {}, "taken": 0, "sum": None})
            g["vals"][rank] = t
            if len(g["vals"]) == size:
                acc = g["vals"][0].clone()
                for r in range(1, size):
                    acc += g["vals"][r]
                g["sum"] = acc
                self._cv.notify_all()
            deadline = time.monotonic() + self.timeout
            while g["sum"] is None:
                left = deadline - time.monotonic()
                if left <= 0:
                    self.stats["timeouts"] += 1
                    arrived = sorted(g["vals"])
                    self._groups.pop(key, None)
                    raise TimeoutError(f"all-reduce '{key}' timed out after {self.timeout}s: arrived ranks {arrived} of {size}")
                self._cv.wait(left)
            g["taken"] += 1
            out = g["sum"]
            if g["taken"] == size:
                self._groups.pop(key, None)
            return out

    def close(self) -> None:
        self._stop = True
        try:
            self._sock.close()
        except OSError:
            pass


class SocketCollectives(Collectives):
    def __init__(self, address, rank: int, size: int, session: str = "default", timeout: float = 60.0):
        self.rank, self.size, self.session = rank, size, session
        self._sock = socket.create_connection(address, timeout=timeout)
        self._sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._seq: dict[str, int] = {}
        self._lock = threading.Lock()

    def all_reduce_sum(self, key: str, t: torch.Tensor) -> torch.Tensor:
        with self._lock:
            n = self._seq.get(key, 0)
            self._seq[key] = n + 1
            wire = f"session:{self.session}:{n}:{key}"
            hdr = json.dumps({"key": wire, "rank": self.rank, "size": self.size}).encode()
            _send_frame(self._sock, MSG_ALLREDUCE, struct.pack("<I", len(hdr)) + hdr + dten.encode(t.float()))
            mtype, body = _recv_frame(self._sock)
        if mtype == MSG_ERROR:
            raise TimeoutError(body.decode(errors="replace"))
        t.copy_(dten.decode(body).to(t.dtype))
        return t

    def close(self) -> None:
        self._sock.close()
