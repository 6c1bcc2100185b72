"""Tensor-parallel identity, shard planning and the collective interface.

Reference behaviour kept: ``enabled = size > 1``, rank 0 is the coordinator rank
(core/.../model/tensorparallel/TensorParallelContext.java:9-40); a size is *compatible* with a model when heads,
KV heads, attention/KV widths and the MLP intermediate all divide evenly, and ``choose_size`` picks the largest compatible
size not above the number of workers (TensorParallelPlanner.java:21-90). The only collective of the reference is
``allReduceSum(key, tensor)`` after ``o_proj`` and ``down_proj`` (TensorParallelCollectives.java:14-58); backends here:

* :class:`SingleRankCollectives` — identity (SingleRankTensorParallelCollectives.java:10-15);
* :class:`TorchCollectives` — ``torch.distributed`` (NCCL on GPUs = baseline path, gloo on CPU);
* :class:`InProcessCollectives` — thread ranks sharing a monitor, for tests without a cluster (the reference's test fake
  core/src/test/.../InProcessTensorParallelCollectives.java);
* the fused GEMM+all-reduce path over peer memory lives in :mod:`deliverance_b200.parallel.fused`.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Optional

import torch

from ..config import ModelConfig


@dataclass(frozen=True)
class ShardRange:
    begin: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


@dataclass(frozen=True)
class TPPlan:
    rank: int
    size: int
    heads: ShardRange
    kv_heads: ShardRange
    intermediate: ShardRange
    hidden: ShardRange


class TensorParallelPlanner:
    @staticmethod
    def compatible(cfg: ModelConfig, size: int) -> bool:
        if size < 1:
            return False
        if size == 1:
            return True
        dims = [cfg.num_heads, cfg.q_size, cfg.hidden_size]
        if cfg.intermediate_size:
            dims.append(cfg.intermediate_size)
        # KV heads either split evenly or, with more ranks than KV heads, are replicated: size / kv_heads ranks share one head
        kv_ok = cfg.num_kv_heads % size == 0 or size % cfg.num_kv_heads == 0
        return kv_ok and all(d % size == 0 for d in dims)

    @staticmethod
    def validate(cfg: ModelConfig, size: int) -> None:
        if not TensorParallelPlanner.compatible(cfg, size):
            raise ValueError(
                f"tensor parallel size {size} does not divide heads={cfg.num_heads}, kv_heads={cfg.num_kv_heads}, "
                f"hidden={cfg.hidden_size}, intermediate={cfg.intermediate_size}")

    @staticmethod
    def choose_size(cfg: ModelConfig, workers: int) -> int:
        for s in range(max(1, workers), 0, -1):
            if TensorParallelPlanner.compatible(cfg, s):
                return s
        return 1

    @staticmethod
    def plan(cfg: ModelConfig, rank: int, size: int) -> TPPlan:
        TensorParallelPlanner.validate(cfg, size)
        if not 0 <= rank < size:
            raise ValueError(f"rank {rank} outside [0, {size})")

        def rng(n: int) -> ShardRange:
            per = n // size
            return ShardRange(rank * per, (rank + 1) * per)

        if cfg.num_kv_heads % size == 0:
            kv = rng(cfg.num_kv_heads)
        else:
            head = rank // (size // cfg.num_kv_heads)
            kv = ShardRange(head, head + 1)
        return TPPlan(rank, size, rng(cfg.num_heads), kv, rng(max(cfg.intermediate_size, size)), rng(cfg.hidden_size))


class Collectives:
    """All-reduce-sum interface. ``key`` names the call site (``layer.N.self_attn.o_proj`` / ``layer.N.mlp.down_proj``)."""

    rank = 0
    size = 1

    def all_reduce_sum(self, key: str, t: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def all_gather(self, t: torch.Tensor) -> list[torch.Tensor]:
        raise NotImplementedError

    def broadcast_object(self, obj, src: int = 0):
        return obj

    def barrier(self) -> None:
        pass

    def close(self) -> None:
        pass


class SingleRankCollectives(Collectives):
    def all_reduce_sum(self, key, t):
        return t

    def all_gather(self, t):
        return [t]


class TorchCollectives(Collectives):
    """``torch.distributed`` process group (NCCL for CUDA tensors, gloo for CPU tensors)."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def all_reduce_sum(self, key, t):
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)
        return t

    def all_gather(self, t):
        outs = [torch.empty_like(t) for _ in range(self.size)]
        self.dist.all_gather(outs, t.contiguous(), group=self.group)
        return outs

    def broadcast_object(self, obj, src=0):
        box = [obj]
        self.dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def barrier(self):
        self.dist.barrier(group=self.group)


class InProcessGroup:
    """Shared monitor for thread ranks: collects ``size`` contributions per key, reduces, hands every caller a copy.
    A wait that exceeds ``timeout`` raises with the key and the ranks that arrived (the reference's collective server
    reports the same diagnostics, HttpTensorParallelCollectiveServer.java:140-156)."""

    def __init__(self, size: int, timeout: float = 30.0):
        if size < 2:
            raise ValueError("an in-process group needs at least 2 ranks")
        self.size = size
        self.timeout = timeout
        self._cv = threading.Condition()
        self._slots: dict[str, dict] = {}
        self._seq: dict[tuple[int, str], int] = {}

    def exchange(self, rank: int, key: str, value):
        with self._cv:
            n = self._seq.get((rank, key), 0)
            self._seq[(rank, key)] = n + 1
            wire = f"{key}#{n}"
            slot = self._slots.setdefault(wire, {"vals": {}, "taken": 0})
            slot["vals"][rank] = value
            if len(slot["vals"]) == self.size:
                self._cv.notify_all()
            deadline = time.monotonic() + self.timeout
            while len(slot["vals"]) < self.size:
                left = deadline - time.monotonic()
                if left <= 0:
                    arrived = sorted(slot["vals"])
                    raise TimeoutError(f"collective '{key}' timed out after {self.timeout}s: arrived ranks {arrived} of {self.size}")
                self._cv.wait(left)
            vals = [slot["vals"][r] for r in range(self.size)]
            slot["taken"] += 1
            if slot["taken"] == self.size:
                del self._slots[wire]
            return vals


class InProcessCollectives(Collectives):
    def __init__(self, group: InProcessGroup, rank: int):
        self.group = group
        self.rank = rank
        self.size = group.size

    def all_reduce_sum(self, key, t):
        vals = self.group.exchange(self.rank, "ar:" + key, t.detach().clone())
        acc = vals[0].clone()
        for v in vals[1:]:
            acc += v
        t.copy_(acc)
        return t

    def all_gather(self, t):
        return [v.clone() for v in self.group.exchange(self.rank, "ag", t.detach().clone())]

    def broadcast_object(self, obj, src=0):
        return self.group.exchange(self.rank, "bc", obj)[src]

    def barrier(self):
        self.group.exchange(self.rank, "barrier", None)


class TensorParallelContext:
    def __init__(self, rank: int = 0, size: int = 1, collectives: Optional[Collectives] = None):
        self.rank = rank
        self.size = size
        self.collectives = collectives or SingleRankCollectives()
        self.fused = None  # set by parallel.fused when peer-memory kernels are available

    @property
    def enabled(self) -> bool:
        return self.size > 1

    @property
    def is_coordinator(self) -> bool:
        return self.rank == 0

    def all_reduce(self, key: str, t: torch.Tensor) -> torch.Tensor:
        if not self.enabled:
            return t
        if self.fused is not None and t.is_cuda:
            return self.fused.all_reduce(t, key)  # one-shot peer-memory kernel for decode-size tensors, NCCL otherwise
        return self.collectives.all_reduce_sum(key, t)


SINGLE = TensorParallelContext()
