"""Fused tensor-parallel paths over NVLink peer memory.

``FusedTensorParallel`` owns one symmetric allocation per rank (``torch.distributed._symmetric_memory``: CUDA virtual-memory
handles exchanged between the ranks of one node, every rank's buffer mapped into every process) that holds the receive
slabs and the flag matrix used by the GEMM kernel's all-reduce epilogue (csrc/gemm_tc.cuh). ``linear_all_reduce`` replaces
the reference's ``allReduceSum`` round trip through a central HTTP/TCP server after ``o_proj`` and ``down_proj``
(core/.../generator/CausalSelfAttention.java:403-405,448-452; core/.../model/tensorparallel/TensorParallelMlp.java:169-171)
with peer stores issued from inside the GEMM epilogue; shapes outside the fused path (grids larger than one wave) fall back
to the GEMM followed by the NCCL all-reduce.

Prefill-size batches (at least 256 rows per rank) have a second path, off unless ``DLV_TP_SCATTER=1``: GEMM -> reduce-scatter
-> all-gather. The GEMM epilogue stores each partial tile into the receive area of the rank that owns those token rows while
the other tiles are still being computed and never waits; a reduce kernel sums the owned rows and pushes them to every
rank's gather area; a last kernel waits for the peers' rows and copies them into the output (``ScatterState``,
csrc/gemm_tc.cuh epilogue 3, csrc/comm.cu). Each rank sends and receives ``2 (n - 1) / n`` of the output over NVLink, the
first half under the GEMM.

Plain peer loads/stores by default; the decode-size sum can optionally go through the NVSwitch (``DLV_TP_REDUCE=nvls``,
``multimem.ld_reduce``). No TMA multicast anywhere. With the default a rank that leaves between steps cannot fault the others
through a multicast binding.
"""
from __future__ import annotations

import torch

from .. import ops
from .context import TensorParallelContext

NCTA_MAX = 1024


def row_cut(M: int, size: int, rank: int) -> tuple:
    """``(rows_per_rank, first, count)``: rank ``rank`` owns token rows ``[first, first + count)`` of an ``M``-row batch; rows per rank
    are ``ceil(M / size)`` rounded up to 8 (the same cut as the extension's ``scatter_plan``)."""
    rpr = -(-(-(-M // size)) // 8) * 8
    first = min(M, rank * rpr)
    return rpr, first, max(0, min(rpr, M - rank * rpr))


def scatter_enabled() -> bool:
    import os

    return os.environ.get("DLV_TP_SCATTER", "0") == "1"


class ScatterState:
    """Symmetric receive / gather areas and counters of the GEMM -> reduce-scatter -> all-gather path."""

    def __init__(self, tp: TensorParallelContext, device, max_rows: int, max_cols: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        pad_rows = max_rows + 8 * tp.size  # rows per rank are rounded up to 8
        self.recv_elems = pad_rows * max_cols
        self.gather_elems = max_rows * max_cols
        recv_bytes, gather_bytes = self.recv_elems * 2, self.gather_elems * 2
        self.buf = symm.empty(recv_bytes + gather_bytes + 128, dtype=torch.uint8, device=device)  # 24 u32 counters, padded
        self.buf[recv_bytes + gather_bytes:].zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.buf, dist.group.WORLD)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.comm = ops.require_ext().TpScatter(tp.rank, tp.size, ptrs, [p + recv_bytes for p in ptrs],
                                                [p + recv_bytes + gather_bytes for p in ptrs], self.recv_elems, self.gather_elems)
        dist.barrier()
        torch.cuda.synchronize(device)


class ExpertAllToAll:
    """Expert-parallel dispatch / return over peer memory for token rows that are sharded over the ranks (csrc/a2a.cu). One instance
    serves every mixture-of-experts layer of a model: ``cap`` = most (token, slot) pairs a rank can send in one forward."""

    def __init__(self, tp: TensorParallelContext, device, n_local_experts: int, hidden: int, cap: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.tp, self.device, self.ne, self.H, self.cap = tp, torch.device(device), n_local_experts, hidden, cap
        recv_b = tp.size * cap * hidden * 2
        meta_b = (tp.size * 2 * n_local_experts * 4 + 15) // 16 * 16
        flag_b = 64
        ret_b = cap * hidden * 2
        self.buf = symm.empty(recv_b + meta_b + flag_b + ret_b, dtype=torch.uint8, device=self.device)
        self.buf[recv_b:recv_b + meta_b + flag_b].zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm.rendezvous(self.buf, dist.group.WORLD)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.ret_local = self.buf[recv_b + meta_b + flag_b:].view(torch.bfloat16).view(cap, hidden)
        self.comm = ops.require_ext().ExpertA2A(tp.rank, tp.size, n_local_experts, cap, hidden, ptrs, [p + recv_b for p in ptrs],
                                                [p + recv_b + meta_b for p in ptrs], [p + recv_b + meta_b + flag_b for p in ptrs])
        self.sent_rows = 0   # rows this rank pushed to other ranks (NVLink traffic = rows * hidden * 2 bytes, the same again on the way back)
        dist.barrier()
        torch.cuda.synchronize(self.device)

    def forward(self, x_own: torch.Tensor, perm: torch.Tensor, offsets: torch.Tensor, k: int, run_experts, max_recv_rows: int):
        """``x_own`` [T_own, H] with ``perm`` / ``offsets`` from the router over the own tokens. ``run_experts(xs, local_offsets)``
        multiplies rows grouped by local expert and returns rows in the same order. Returns the return buffer: expert outputs of
        this rank's (token, slot) pairs at their grouped row index (the layout ``moe_combine`` expects)."""
        self.comm.dispatch(x_own.contiguous(), perm, offsets, k)
        xs, local_offsets, seg = self.comm.receive(max_recv_rows, x_own)
        ys = run_experts(xs, local_offsets)
        ops._count(7)
        return self.comm.finish(ys.contiguous(), local_offsets, seg, self.ret_local)


class FusedTensorParallel:
    def __init__(self, tp: TensorParallelContext, device, max_rows: int = 128, max_cols: int = 8192):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.tp = tp
        self.device = torch.device(device)
        self.slab = max_rows * max_cols
        recv_bytes = 2 * tp.size * self.slab * 2
        flag_bytes = tp.size * NCTA_MAX * 4
        self.recv_bytes = recv_bytes
        total = recv_bytes + flag_bytes
        self.buf = symm.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm.rendezvous(self.buf, dist.group.WORLD)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rounds = torch.zeros(NCTA_MAX, dtype=torch.int32, device=self.device)
        self.call = torch.zeros(2, dtype=torch.int32, device=self.device)
        e = ops.require_ext()
        self.comm = e.TpComm(tp.rank, tp.size, ptrs, [p + recv_bytes for p in ptrs], self.slab, NCTA_MAX, self.rounds, self.call)
        # How a decode-size row-parallel projection is summed (DLV_TP_REDUCE): "epilogue" (default) = wait for the peers and sum inside
        # the GEMM epilogue, the residual add + norm is the next kernel; "split" = the GEMM epilogue stores its partial tiles into every
        # rank's slab and leaves, a row-wise kernel waits for the ranks, sums them and applies the residual add + norm; "nvls" = the
        # same with the sum done by the NVSwitch (multimem.ld_reduce on the multicast address; falls back to "split" when the
        # allocation has no multicast binding). Measured per projection + norm at 64 tokens (8 ranks / 2 ranks): epilogue 29.0 / 29.4 us,
        # split 32.7 / 28.8 us, nvls 33.7 / 34.0 us, GEMM + NCCL all-reduce + norm 38.9 / 92.9 us; whole decode step at 8 ranks 3.45 /
        # 3.56 / 3.41 ms: the three forms tie, so the one with the fewest launches is the default. Tests in which a rank leaves between
        # steps must not run "nvls" (a multicast binding of a dead rank faults the others).
        import os

        self.reduce_mode = os.environ.get("DLV_TP_REDUCE", "epilogue")
        self.push_mode = 1
        if self.reduce_mode == "nvls":
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            if mc:
                self.comm.set_multicast(mc)
                self.push_mode = 2
            else:
                self.reduce_mode = "split"
        dist.barrier()
        torch.cuda.synchronize(self.device)
        self.stats = {"fused": 0, "fallback": 0, "scatter": 0, "split": 0}
        self.scatter = None
        if scatter_enabled():
            import os

            self.scatter = ScatterState(tp, self.device, int(os.environ.get("DLV_TP_SCATTER_ROWS", "8192")), max_cols)

    @staticmethod
    def create(tp: TensorParallelContext, device) -> "FusedTensorParallel":
        if tp.size < 2 or tp.size > 8:
            raise ValueError("fused tensor parallelism needs 2..8 ranks on one node")
        return FusedTensorParallel(tp, device)

    def linear_all_reduce(self, x: torch.Tensor, w, key: str) -> torch.Tensor:
        """``all_reduce_sum(x @ W_shard^T)`` with the sum fused into the GEMM epilogue when the shape allows it."""
        out = torch.empty(x.shape[0], w.N, dtype=torch.bfloat16, device=x.device)
        bias = w.bias  # added once, after the sum, by the reducing epilogue of every rank
        if x.shape[0] > 0 and w.handle().run_tp(x, out, self.comm, bias):
            ops._count()
            self.stats["fused"] += 1
            return out
        if self.scatter is not None and x.shape[0] >= 256 * self.tp.size and not torch.cuda.is_current_stream_capturing():
            if w.handle().run_scatter(x, out, self.scatter.comm, bias):
                ops._count(3)
                self.stats["scatter"] += 1
                return out
        self.stats["fallback"] += 1
        y = ops.linear(x, w) if self.tp.rank == 0 or w.bias is None else ops.linear(x, _no_bias(w))
        return self.tp.collectives.all_reduce_sum(key, y)


    def expert_a2a(self, n_local_experts: int, hidden: int, k: int):
        """The all-to-all state for a model's mixture-of-experts layers (created on first use; every rank must call it at the same
        point). Sized for the largest sequence-parallel batch: ``DLV_TP_SCATTER_ROWS`` rows cut over the ranks, ``k`` slots each."""
        key = (n_local_experts, hidden, k)
        cache = self.__dict__.setdefault("_a2a", {})
        if key not in cache:
            import os

            rows = int(os.environ.get("DLV_TP_SCATTER_ROWS", "8192"))
            cache[key] = ExpertAllToAll(self.tp, self.device, n_local_experts, hidden, (row_cut(rows, self.tp.size, 0)[0] + 8) * k)
        return cache[key]

    def linear_reduce_norm(self, x: torch.Tensor, w, residual: torch.Tensor, norm_w: torch.Tensor, post_w, eps: float, offset: float,
                           res_mult: float):
        """Row-parallel projection, tensor-parallel sum, residual add and RMSNorm as two kernels: the GEMM publishes its partial
        tiles and leaves, a row-wise kernel waits for the ranks (so the wait is not inside the GEMM's CTAs and the next GEMM's weight
        stream runs underneath), sums them in rank order (or through the NVSwitch), adds into ``residual`` (in place) and returns
        ``rmsnorm(residual, norm_w)``. Returns ``None`` (nothing launched) when the shape is outside this path or it is switched off."""
        M = x.shape[0]
        if self.reduce_mode == "epilogue" or M == 0 or M > 128 or w.N % 8 or w.N > 12288 or not residual.is_contiguous():
            return None
        ctas = w.handle().run_tp_push(x, self.comm, self.push_mode)
        if ctas == 0:
            return None
        out = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
        ops.require_ext().tp_reduce_norm(self.comm, self.push_mode, ctas, M, w.N, 1, w.bias, residual, post_w, norm_w, out, eps, offset, res_mult)
        ops._count(2)
        self.stats["split"] += 1
        return out

    def linear_reduce_scatter(self, x: torch.Tensor, w, key: str) -> torch.Tensor:
        """Rows ``own_rows(M)`` of ``sum over ranks (x @ W_shard^T)``: the GEMM epilogue sends every partial tile to the rank that
        owns its token rows, the owner sums. Sequence-parallel building block: follow it with ``all_gather_linear(..., ordered=
        True)`` (which also orders the ranks before the next scatter). Outside the peer-memory path: all-reduce, then slice."""
        M = x.shape[0]
        first, count = self.own_rows(M)
        if self.scatter is not None and M >= 256 * self.tp.size and not torch.cuda.is_current_stream_capturing():
            out = torch.empty(count, w.N, dtype=torch.bfloat16, device=x.device)
            if w.handle().run_scatter(x, out, self.scatter.comm, w.bias, False):
                ops._count(2)
                self.stats["scatter"] += 1
                return out
        return self.linear_all_reduce(x, w, key)[first:first + count]

    def own_rows(self, M: int) -> tuple:
        """``(first, count)``: the token rows of an ``M``-row batch this rank owns in the scatter / gather paths."""
        _, first, count = row_cut(M, self.tp.size, self.tp.rank)
        return first, count

    def all_gather_linear(self, x_own: torch.Tensor, M: int, w, ordered: bool = False) -> torch.Tensor:
        """``all_gather(x) @ W_shard^T`` for activations whose rows are sharded over the ranks (``x_own`` = the rows of
        ``own_rows(M)``). The rows are pushed into every rank's gather area and the GEMM waits per token tile for their owners,
        so weights stream and arrived tiles run under the transfer. ``ordered``: the caller guarantees that every rank has
        finished the previous consumer of the gather area (a reduce-scatter in between does); otherwise a barrier is issued."""
        out = torch.empty(M, w.N, dtype=torch.bfloat16, device=x_own.device)
        if self.scatter is not None and not torch.cuda.is_current_stream_capturing():
            if not ordered:
                self.tp.collectives.all_reduce_sum("ag.order", torch.zeros(1, device=x_own.device))
            if w.handle().run_gathered(x_own.contiguous(), M, out, self.scatter.comm, w.bias):
                ops._count(2)
                self.stats["gathered"] = self.stats.get("gathered", 0) + 1
                return out
        self.stats["fallback"] += 1
        # ranks hold blocks of rows_per_rank rows, only the tail of the last non-empty block is padding
        full = torch.cat(self.tp.collectives.all_gather(_pad_rows(x_own, self._rows_per_rank(M))), dim=0)[:M]
        return ops.linear(full, w)

    def _rows_per_rank(self, M: int) -> int:
        return row_cut(M, self.tp.size, self.tp.rank)[0]

    def all_reduce(self, x: torch.Tensor, key: str) -> torch.Tensor:
        """Sum a small bf16 ``[rows, H]`` tensor over the ranks with the one-shot peer-memory kernel, NCCL otherwise."""
        if x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous():
            out = torch.empty_like(x)
            if ops.require_ext().oneshot_allreduce(x, self.comm, out):
                ops._count()
                self.stats["fused"] += 1
                return out
        self.stats["fallback"] += 1
        return self.tp.collectives.all_reduce_sum(key, x)

    def moe_combine_all_reduce(self, ys, pos, w, T: int, k: int, offsets, e0: int, ne: int):
        """Top-k weighted combine of the local experts' rows fused with the sum over the expert-parallel ranks. Returns ``None``
        when the batch is outside the fused path (the caller then combines locally and all-reduces)."""
        out = torch.empty(T, ys.shape[1], dtype=torch.bfloat16, device=ys.device)
        if ops.require_ext().moe_combine_allreduce(ys, pos, w, T, k, offsets, e0, ne, self.comm, out):
            ops._count()
            self.stats["fused"] += 1
            return out
        return None


def _pad_rows(x: torch.Tensor, rows: int) -> torch.Tensor:
    if x.shape[0] == rows:
        return x.contiguous()
    return torch.cat([x, x.new_zeros(rows - x.shape[0], x.shape[1])], dim=0)


def _no_bias(w):
    import copy

    c = copy.copy(w)
    c.bias = None
    c._handle = w._handle
    return c
