"""Mixture-of-experts feed-forward for mixtral, qwen3_moe and granitemoehybrid.

Routing conventions (reference): Mixtral — softmax over all experts, top-k, renormalise
(core/.../model/MixtureOfExpertsBlock.java:100-112); Qwen3-MoE — softmax over all, top-k, renormalise only with
``norm_topk_prob`` (core/.../model/qwen3/Qwen3MoeFeedForward.java:276-301); Granite — top-k on the logits, softmax over
the k (GraniteMoeHybridMoeFeedForward.java:112-141). Tokens are grouped by expert, each expert runs gate|up -> act*mul ->
down on its rows, and results are scatter-added with the route weight (Qwen3MoeFeedForward.java:107-183).

On CUDA the router (softmax/top-k/renorm + per-expert histogram and row offsets) and the gather / weighted scatter are
single kernels (csrc/moe.cu) and each expert GEMM is a tcgen05 launch on its contiguous row group.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..ops import ref


_SM_COUNT = 148  # B200
_ROUTE_ONE_LAUNCH = [os.environ.get("DLV_MOE_ROUTE", "fused") != "split"]  # decode-size routing in one launch ("split": the separate kernels)


def moe_forward(model, i: int, lw, x: torch.Tensor) -> torch.Tensor:
    """Routed experts of one layer. Under tensor parallelism the experts are split across ranks when their count divides
    (expert parallelism: tokens are replicated after the attention all-reduce, so dispatch is a local selection and the
    combine is a sum over ranks); otherwise every rank holds all experts and no communication is needed."""
    cfg = model.cfg
    E, k = cfg.num_experts, cfg.experts_per_token
    logits = ops.linear(x, lw.router, out_f32=True)
    renorm = True if cfg.model_type == "mixtral" else (cfg.norm_topk_prob if cfg.router_mode == "softmax_topk" else False)
    e0, ne = lw.expert0, lw.n_local_experts or E
    if x.device.type == "cuda":
        y, reduced = _moe_cuda(model, lw, x, logits, E, k, cfg.router_mode, renorm, cfg.hidden_act, e0, ne)
        if reduced:
            return y
    else:
        w, idx = ref.moe_route(logits, k, cfg.router_mode, renorm)
        local = (idx >= e0) & (idx < e0 + ne)
        y = ref.moe_experts(
            x, torch.where(local, w, torch.zeros_like(w)), torch.where(local, idx - e0, torch.full_like(idx, -1)),
            lambda e, rows: ops.linear(rows, lw.experts_gate_up[e]),
            lambda e, h: ops.linear(h, lw.experts_down[e]),
            ne, cfg.hidden_act,
            (lambda e, rows: ops.linear_act(rows, lw.experts_gate_up[e], cfg.hidden_act)) if lw.fused_act_experts else None,
        )
    if ne != E:
        y = model.tp.all_reduce(f"layer.{i}.moe.combine", y)
    return y


def moe_forward_sharded(model, i: int, lw, x_own: torch.Tensor, a2a, total_rows: int) -> torch.Tensor:
    """Routed experts for token rows that are sharded over the ranks (sequence-parallel forward) with expert parallelism: every rank
    routes its own rows, an all-to-all over peer memory carries each (token, slot) row to the rank that owns its expert, the grouped
    expert GEMMs run there, the outputs travel back and are combined with the route weights (``parallel.fused.ExpertAllToAll``).
    ``total_rows``: token rows of the whole batch (bounds what one rank can receive)."""
    cfg = model.cfg
    E, k = cfg.num_experts, cfg.experts_per_token
    e = ops.require_ext()
    ne = lw.n_local_experts
    renorm = True if cfg.model_type == "mixtral" else (cfg.norm_topk_prob if cfg.router_mode == "softmax_topk" else False)
    T = x_own.shape[0]
    logits = ops.linear(x_own, lw.router, out_f32=True) if T else torch.zeros(0, E, device=x_own.device)
    w, idx, counts, offsets, perm, pos = e.moe_route(logits.contiguous(), k, 0 if cfg.router_mode == "softmax_topk" else 1, bool(renorm))
    ops._count(2)
    max_recv = min(total_rows * k, a2a.cap * model.tp.size)
    bn = ops.moe_token_tile(max(1, total_rows * k // model.tp.size), ne, lw.experts_gate_up_grouped.q4)
    if lw.fused_act_experts:
        bn = max(bn, 16)
    max_items = max(1, (max_recv + bn - 1) // bn + ne)
    gu_w, down_w = lw.experts_gate_up_grouped, lw.experts_down_grouped

    def run_experts(xs, local_offsets):
        items = e.moe_items(local_offsets, 0, ne, bn, max_items)
        ops._count()
        if lw.fused_act_experts and bn >= 16:
            hmid = gu_w.run_act(xs, items, bn, 1, cfg.hidden_act)
        else:
            hmid = ops.act_mul(gu_w.run(xs, items, bn, 1), cfg.hidden_act)
        return down_w.run(hmid, items, bn, 1)

    ret = a2a.forward(x_own, perm, offsets, k, run_experts, max_recv)
    a2a.sent_rows += int(T * k)
    if T == 0:
        return x_own
    ops._count()
    return e.moe_combine(ret[: T * k], pos, w, T, k)


def _moe_cuda(model, lw, x, logits, E, k, mode, renorm, act, e0, ne):
    e = ops.require_ext()
    st = model._stage
    T, H = x.shape
    rows = T * k
    ep = ne != E
    bn = ops.moe_token_tile(rows if not ep else max(1, rows * ne // E), ne, lw.experts_gate_up_grouped.q4)
    if lw.fused_act_experts:
        bn = max(bn, 16)  # interleaved expert rows exist for the tensor-core grouped GEMM's epilogue only
    max_items = min((rows + bn - 1) // bn + ne, rows) if rows >= ne else rows
    max_items = max(1, max_items)
    rng = None
    xs = None
    with st("moe.route"):
        # weights [T, k] fp32, expert ids [T, k], counts [E], offsets [E + 1], perm: grouped row -> (token * k + slot), pos: inverse,
        # items: the grouped GEMM's work list. Decode-size batches get all of it from one launch.
        mode_i = 0 if mode == "softmax_topk" else 1
        routed = e.moe_route_items(logits.contiguous(), k, mode_i, bool(renorm), e0, ne, bn, max_items) if _ROUTE_ONE_LAUNCH[0] else []
        if routed:
            w, idx, counts, offsets, perm, pos, items = routed
            ops._count()
        else:
            w, idx, counts, offsets, perm, pos = e.moe_route(logits.contiguous(), k, mode_i, bool(renorm))
            items = e.moe_items(offsets, e0, ne, bn, max_items)
            ops._count(3)
        rng = (offsets, e0, ne) if ep else (None, 0, 0)

    def gathered():
        """x rows in expert-grouped order [T * k, H] (only the local experts' rows are filled)."""
        ops._count()
        return e.moe_gather(x, perm, k, *rng)

    gu_w, down_w = lw.experts_gate_up_grouped, lw.experts_down_grouped
    small = bn <= 64  # decode-sized groups: split K so that more CTAs stream weights

    def k_splits(wt) -> int:
        """Split K only as far as the grid needs it: every split pays the tile's set-up and a reduction again, so a projection whose
        (local experts x 128-row tiles) already fill two waves of the GPU runs unsplit."""
        if not small:
            return 1
        tiles = max(1, ne) * ((wt.N + 127) // 128)
        want = (2 * _SM_COUNT + tiles - 1) // tiles
        return max(1, min(8, wt.K // 1024, want))

    if lw.fused_act_experts and bn >= 16:
        with st("moe.gate_up"):  # act(gate) * up in the grouped GEMM's epilogue (interleaved expert rows)
            hmid = gu_w.run_act(gathered(), items, bn, k_splits(gu_w), act)
    else:
        if lw.fused_act_experts:
            raise RuntimeError("interleaved expert weights need the tensor-core grouped GEMM (token tile >= 16)")
        hmid = None
        if bn <= 8:
            # a handful of rows per expert: grouped GEMV with the gated activation in its epilogue; it reads the token rows through
            # the permutation, so the copy into expert order is skipped
            with st("moe.gate_up"):
                hmid = gu_w.run_gemv_act(x, items, act, perm, k)
        if hmid is None:
            with st("moe.gate_up"):
                xs = gathered()
                gu = gu_w.run(xs, items, bn, k_splits(gu_w))
            with st("moe.activation_multiply"):
                hmid = ops.act_mul(gu, act)
    with st("moe.down"):
        ys = down_w.run(hmid, items, bn, k_splits(down_w))
    with st("moe.combine"):
        fused = getattr(model.tp, "fused", None)
        if ep and fused is not None:
            y = fused.moe_combine_all_reduce(ys, pos, w, T, k, offsets, e0, ne)  # combine + sum over ranks in one kernel
            if y is not None:
                return y, True
        ops._count()
        return e.moe_combine(ys, pos, w, T, k, *rng), False
