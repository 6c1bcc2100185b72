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
        meta = _chunk_meta(batch, x.device)
        ops._count(5 if not meta["multi"] else 7)
        y = e.mamba2_forward(zx, m["conv_w"].reshape(-1), m["conv_b"], m["dt_bias"], m["A_log"], m["D"], m["norm_w"], conv_state, ssm_state,
                             batch.state_slots, batch.q_start, batch.q_len, batch.positions, meta["row_seq"], meta["chunk_seq"],
                             meta["chunk_row0"], meta["chunk_len"], meta["chunk_first"], meta["chunk_last"], meta["seq_chunk0"],
                             meta["seq_nchunks"], meta["multi"], cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_n_groups, cfg.mamba_d_state,
                             cfg.norm_eps)
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


CHUNK = 128


def _chunk_meta(batch, device) -> dict:
    """Index tensors of the chunked scan (cached on the batch). Decode batches build them with device ops only, so the
    step stays capturable in a CUDA graph."""
    cached = getattr(batch, "_mamba_meta", None)
    if cached is not None:
        return cached
    i32 = dict(dtype=torch.int32, device=device)
    if batch.is_decode:
        n = batch.num_seqs
        ar = torch.arange(n, **i32)
        one = torch.ones(n, **i32)
        meta = {"row_seq": ar, "chunk_seq": ar, "chunk_row0": ar, "chunk_len": one, "chunk_first": one, "chunk_last": one,
                "seq_chunk0": ar, "seq_nchunks": one, "multi": False}
    else:
        qs, ql = batch.q_start.tolist(), (batch.q_len_host or batch.q_len.tolist())
        row_seq, cseq, crow, clen, cfirst, clast, s0, sn = [], [], [], [], [], [], [], []
        for s, (a, n) in enumerate(zip(qs, ql)):
            row_seq += [s] * n
            s0.append(len(cseq))
            nc = max(1, (n + CHUNK - 1) // CHUNK)
            sn.append(nc)
            for c in range(nc):
                cseq.append(s)
                crow.append(a + c * CHUNK)
                clen.append(max(0, min(CHUNK, n - c * CHUNK)))
                cfirst.append(1 if c == 0 else 0)
                clast.append(1 if c == nc - 1 else 0)
        t = lambda v: torch.tensor(v, dtype=torch.int32).to(device)  # noqa: E731
        meta = {"row_seq": t(row_seq), "chunk_seq": t(cseq), "chunk_row0": t(crow), "chunk_len": t(clen), "chunk_first": t(cfirst),
                "chunk_last": t(clast), "seq_chunk0": t(s0), "seq_nchunks": t(sn), "multi": any(v > 1 for v in sn)}
    batch._mamba_meta = meta
    return meta
