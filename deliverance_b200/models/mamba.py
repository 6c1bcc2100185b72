"""Mamba2 mixer layer of granitemoehybrid.

in_proj -> split ``[gate (I) | x (I) | B (G*S) | C (G*S) | dt (H)]`` -> ``dt = softplus(dt + dt_bias)`` -> causal depthwise
conv1d with a rolling state + SiLU -> SSM recurrence ``h = h * exp(dt*A) + B * dt * x``, ``y = C.h + D*x`` -> ``y *= silu(gate)``
-> RMSNorm over the whole intermediate -> out_proj (reference: core/.../model/granitemoehybrid/GraniteMoeHybridMambaLayer.java:
130-252; the reference walks tokens one by one). Per-sequence conv / SSM state lives in the KV manager's state slots and is
reset when a sequence starts at position 0. On CUDA the scan runs chunked (csrc/mamba.cu): intra-chunk work is
parallel over (head, d_head) with the state carried across chunks; decode is the single-token variant of the same kernel.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import ref


def mamba_forward(model, i: int, lw, x: torch.Tensor, batch, kv) -> torch.Tensor:
    cfg = model.cfg
    m = lw.mamba
    zx = ops.linear(x, m["in_proj"], out_f32=False)
    conv_state, ssm_state = kv.conv_state[i], kv.ssm_state[i]
    I = cfg.mamba_intermediate
    if x.device.type == "cuda":
        e = ops.require_ext()
        y = e.mamba2_forward(zx, m["conv_w"], m["conv_b"], m["dt_bias"], m["A_log"], m["D"], m["norm_w"], conv_state, ssm_state,
                             batch.state_slots, batch.q_start, batch.q_len, batch.positions, cfg.mamba_n_heads, cfg.mamba_d_head,
                             cfg.mamba_n_groups, cfg.mamba_d_state, cfg.norm_eps)
        return ops.linear(y, m["out_proj"])
    out = torch.empty(x.shape[0], I, dtype=torch.float32)
    qs, ql = batch.q_start.tolist(), batch.q_len.tolist()
    slots = batch.state_slots.tolist()
    starts = [int(batch.positions[s]) for s in qs]
    for s, (a, n) in enumerate(zip(qs, ql)):
        if n == 0:
            continue
        slot = slots[s]
        if starts[s] == 0:
            conv_state[slot].zero_()
            ssm_state[slot].zero_()
        out[a : a + n] = ref.mamba2_sequential(zx[a : a + n], m["conv_w"], m["conv_b"], m["dt_bias"], m["A_log"], m["D"], m["norm_w"],
                                               cfg.norm_eps, cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_n_groups, cfg.mamba_d_state,
                                               conv_state[slot], ssm_state[slot], "silu")
    return ops.linear(out.to(x.dtype), m["out_proj"])
