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

import torch

from .. import ops
from ..ops import ref


def moe_forward(model, i: int, lw, x: torch.Tensor) -> torch.Tensor:
    cfg = model.cfg
    E, k = cfg.num_experts, cfg.experts_per_token
    logits = ops.linear(x, lw.router, out_f32=True)
    renorm = True if cfg.model_type == "mixtral" else (cfg.norm_topk_prob if cfg.router_mode == "softmax_topk" else False)
    if x.device.type == "cuda":
        return _moe_cuda(model, lw, x, logits, E, k, cfg.router_mode, renorm, cfg.hidden_act)
    w, idx = ref.moe_route(logits, k, cfg.router_mode, renorm)
    return ref.moe_experts(
        x, w, idx,
        lambda e, rows: ops.linear(rows, lw.experts_gate_up[e]),
        lambda e, h: ops.linear(h, lw.experts_down[e]),
        E, cfg.hidden_act,
    )


def _moe_cuda(model, lw, x, logits, E, k, mode, renorm, act):
    e = ops.require_ext()
    T, H = x.shape
    # weights [T, k] fp32, expert ids [T, k], counts [E], offsets [E + 1], perm: grouped row -> (token * k + slot), pos: inverse
    w, idx, counts, offsets, perm, pos = e.moe_route(logits.contiguous(), k, 0 if mode == "softmax_topk" else 1, bool(renorm))
    ops._count(2)
    xs = e.moe_gather(x, perm, k)  # [T * k, H] rows grouped by expert
    ops._count()
    counts_h = counts.tolist()  # one small D2H per MoE layer; the per-expert launch list needs host row counts
    inter = lw.experts_gate_up[0].N // 2
    hmid = torch.empty(T * k, inter, dtype=x.dtype, device=x.device)
    ys = torch.empty(T * k, H, dtype=x.dtype, device=x.device)
    row = 0
    for ex in range(E):
        n = counts_h[ex]
        if n == 0:
            continue
        gu = ops.linear(xs[row : row + n], lw.experts_gate_up[ex])
        hmid[row : row + n] = ops.act_mul(gu, act)
        ops.linear(hmid[row : row + n], lw.experts_down[ex], out=ys[row : row + n])
        row += n
    ops._count()
    return e.moe_combine(ys, pos, w, T, k)
