"""Plain PyTorch statement of every op in the kernel set.

This is the slow, always-available oracle: the CUDA kernels in ``csrc/`` are tested against these functions evaluated
in fp32, and the CPU execution path of the framework (tests, the fp32 llama oracle) runs on them directly. Math follows
the reference: RMSNorm ``(offset + w) * x * rsqrt(mean(x^2) + eps)`` (core/.../generator/RmsNorm.java:107-121), HF
half-rotation RoPE with pairs ``(i, i + d/2)`` (CausalSelfAttention.java:340-372,429-446), scores
``softmax(softcap(scale * q.k))`` with causal visibility ``j <= pos`` (VectorTensorMathUtils.java:34-78), activations
(math/.../ActivationFunction.java:8-33).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from ..ckpt.jq4 import q4_dequantize


def act_fn(name: str):
    name = (name or "silu").lower()
    if name in ("silu", "swish"):
        return F.silu
    if name in ("gelu_pytorch_tanh", "gelu_new", "gelu_tanh", "gelu_fast"):
        return lambda x: F.gelu(x, approximate="tanh")
    if name == "gelu":
        return F.gelu
    if name == "relu":
        return F.relu
    if name == "tanh":
        return torch.tanh
    raise ValueError(f"unknown activation '{name}'")


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    var = xf.double().pow(2).mean(dim=-1, keepdim=True).float() if x.device.type == "cpu" else xf.pow(2).mean(dim=-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps) * (w.float() + offset)
    return y.to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float, offset: float = 0.0,
                res_mult: float = 1.0) -> torch.Tensor:
    """``residual += x * res_mult`` (in place) and return ``rmsnorm(residual)``."""
    residual.copy_((residual.float() + x.float() * res_mult).to(residual.dtype))
    return rmsnorm(residual, w, eps, offset)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)


def linear_dense(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def linear_q4(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return linear_dense(x, q4_dequantize(packed, scales, torch.float32), bias)


def rope_tables(head_dim: int, max_pos: int, theta: float, factor: float = 1.0, rot_dim: Optional[int] = None):
    """cos/sin tables ``[max_pos, rot/2]`` fp32: angle = pos * theta^(-2i/rot) / factor (math/.../VectorMathUtils.java:20-41)."""
    rot = rot_dim or head_dim
    i = torch.arange(0, rot // 2, dtype=torch.float64)
    inv = 1.0 / (theta ** (2.0 * i / rot)) / factor
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
    return torch.cos(ang).float(), torch.sin(ang).float()


def apply_rope(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[T, heads, d]``; rotates the first ``2 * cos.shape[1]`` dims with pairs (i, i + half)."""
    half = cos.shape[1]
    c = cos[pos].unsqueeze(1).float()
    s = sin[pos].unsqueeze(1).float()
    xf = x.float()
    a, b, rest = xf[..., :half], xf[..., half : 2 * half], xf[..., 2 * half :]
    out = torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)
    return out.to(x.dtype)


def qk_prepare_and_cache(qkv, positions, slots, n_heads, n_kv, head_dim, q_norm_w, k_norm_w, eps, norm_offset,
                         cos, sin, k_cache, v_cache):
    """Split fused qkv ``[T, (H + 2 KV) * D]``, apply optional per-head RMSNorm to q and k, RoPE to q and k, and
    scatter k, v into the paged cache rows ``slots`` (flat row = block * block_size + offset).

    ``k_cache`` / ``v_cache``: ``[num_blocks, KV, block_size, D]``. Returns q ``[T, H, D]``.
    """
    T = qkv.shape[0]
    q, k, v = qkv.split([n_heads * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
    q = q.reshape(T, n_heads, head_dim)
    k = k.reshape(T, n_kv, head_dim)
    v = v.reshape(T, n_kv, head_dim)
    if q_norm_w is not None:
        q = rmsnorm(q, q_norm_w, eps, norm_offset)
        k = rmsnorm(k, k_norm_w, eps, norm_offset)
    if cos is not None:
        q = apply_rope(q, positions, cos, sin)
        k = apply_rope(k, positions, cos, sin)
    nb, kvh, bs, d = k_cache.shape
    blk = torch.div(slots, bs, rounding_mode="floor")
    off = slots % bs
    k_cache[blk, :, off, :] = k.to(k_cache.dtype)
    v_cache[blk, :, off, :] = v.to(v_cache.dtype)
    return q.contiguous()


def paged_attention(q, k_cache, v_cache, block_tables, q_start, q_len, ctx_len, scale, softcap=0.0, window=0,
                    causal=True):
    """Attention of ragged query rows against paged K/V.

    q ``[T, H, D]``; sequence ``i`` owns query rows ``[q_start[i], q_start[i] + q_len[i])`` which are the *last*
    ``q_len[i]`` positions of a context of ``ctx_len[i]`` cached tokens. Row at position ``p`` sees keys ``j <= p``
    (and ``j > p - window`` when ``window > 0``). Score = ``softmax(softcap * tanh(scale * q.k / softcap))``.
    """
    T, H, D = q.shape
    nb, KV, bs, _ = k_cache.shape
    group = H // KV
    out = torch.zeros_like(q)
    for i in range(len(q_len)):
        ql, cl, qs = int(q_len[i]), int(ctx_len[i]), int(q_start[i])
        if ql == 0:
            continue
        nblk = (cl + bs - 1) // bs
        blocks = block_tables[i, :nblk].long()
        k = k_cache[blocks].permute(1, 0, 2, 3).reshape(KV, nblk * bs, D)[:, :cl].float()
        v = v_cache[blocks].permute(1, 0, 2, 3).reshape(KV, nblk * bs, D)[:, :cl].float()
        qi = q[qs : qs + ql].float().permute(1, 0, 2)  # H, ql, D
        k = k.repeat_interleave(group, dim=0)
        v = v.repeat_interleave(group, dim=0)
        s = torch.matmul(qi, k.transpose(1, 2)) * scale
        if softcap and softcap > 0:
            s = torch.tanh(s / softcap) * softcap
        pos = torch.arange(cl - ql, cl, device=q.device).unsqueeze(1)
        j = torch.arange(cl, device=q.device).unsqueeze(0)
        mask = torch.ones(ql, cl, dtype=torch.bool, device=q.device)
        if causal:
            mask &= j <= pos
        if window and window > 0:
            mask &= j > pos - window
        s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs : qs + ql] = torch.matmul(p, v).permute(1, 0, 2).to(q.dtype)
    return out


def act_mul(gate_up: torch.Tensor, act: str) -> torch.Tensor:
    """``act(x[:, :I]) * x[:, I:]`` on a concatenated gate|up projection."""
    I = gate_up.shape[-1] // 2
    g, u = gate_up[..., :I].float(), gate_up[..., I:].float()
    return (act_fn(act)(g) * u).to(gate_up.dtype)


def embedding(table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    out = table[ids.long()].float() * scale
    return out.to(dtype or table.dtype)


def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    return torch.tanh(logits / cap) * cap if cap and cap > 0 else logits


# ---- MoE -------------------------------------------------------------------------------------------------------------
def moe_route(router_logits: torch.Tensor, k: int, mode: str, renorm: bool):
    """Return (weights ``[T, k]`` fp32, expert ids ``[T, k]``).

    ``softmax_topk``: softmax over all experts, take top-k, optionally renormalise (Mixtral always renormalises,
    MixtureOfExpertsBlock.java:100-112; Qwen3-MoE by ``norm_topk_prob``, Qwen3MoeFeedForward.java:276-301).
    ``topk_softmax``: take the top-k logits, softmax over those k (GraniteMoeHybridMoeFeedForward.java:112-141).
    """
    lf = router_logits.float()
    if mode == "softmax_topk":
        p = torch.softmax(lf, dim=-1)
        w, idx = torch.topk(p, k, dim=-1)
        if renorm:
            w = w / w.sum(dim=-1, keepdim=True)
    elif mode == "topk_softmax":
        top, idx = torch.topk(lf, k, dim=-1)
        w = torch.softmax(top, dim=-1)
    else:
        raise ValueError(mode)
    return w, idx


def moe_experts(x, weights, idx, gate_up_fn, down_fn, num_experts, act, gated_fn=None):
    """Group tokens by expert, run gate|up -> act*mul -> down per expert, scatter-add with the route weight. ``gated_fn(e, rows)``
    replaces gate|up + act*mul when the expert weights are stored in the interleaved layout of the fused epilogue."""
    T, Hd = x.shape
    out = torch.zeros(T, Hd, dtype=torch.float32, device=x.device)
    for e in range(num_experts):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = gated_fn(e, x[tok]) if gated_fn is not None else act_mul(gate_up_fn(e, x[tok]), act)
        y = down_fn(e, h).float()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(1))
    return out.to(x.dtype)


# ---- Mamba2 ----------------------------------------------------------------------------------------------------------
def mamba2_sequential(zxbcdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, eps, n_heads, d_head, n_groups, d_state,
                      conv_state, ssm_state, act="silu"):
    """Token-by-token Mamba2 mixer core for ONE sequence (reference GraniteMoeHybridMambaLayer.java:130-252).

    zxbcdt ``[T, I + convDim + H]`` laid out ``[gate (I) | x (I) | B (G*S) | C (G*S) | dt (H)]``;
    conv_state ``[convDim, K-1]``, ssm_state ``[H, d_head, S]`` are updated in place. Returns ``[T, I]`` (after the
    gated RMSNorm over the whole intermediate), fp32 math.
    """
    T = zxbcdt.shape[0]
    I = n_heads * d_head
    GS = n_groups * d_state
    conv_dim = I + 2 * GS
    Kc = conv_w.shape[-1]
    f = act_fn(act)
    A = -torch.exp(A_log.float())
    out = torch.empty(T, I, dtype=torch.float32, device=zxbcdt.device)
    cw = conv_w.float().reshape(conv_dim, Kc)
    for t in range(T):
        row = zxbcdt[t].float()
        gate = row[:I]
        xbc = row[I : I + conv_dim]
        dt = F.softplus(row[I + conv_dim :] + dt_bias.float())
        window = torch.cat([conv_state.float(), xbc.unsqueeze(1)], dim=1)  # convDim, K
        conv = (window * cw).sum(dim=1)
        if conv_b is not None:
            conv = conv + conv_b.float()
        conv_state.copy_(window[:, 1:].to(conv_state.dtype))
        conv = f(conv)
        x = conv[:I].reshape(n_heads, d_head)
        B = conv[I : I + GS].reshape(n_groups, d_state)
        C = conv[I + GS :].reshape(n_groups, d_state)
        hpg = n_heads // n_groups
        Bh = B.repeat_interleave(hpg, dim=0)  # H, S
        Ch = C.repeat_interleave(hpg, dim=0)
        decay = torch.exp(dt * A)  # H
        st = ssm_state.float() * decay.view(-1, 1, 1) + (dt.view(-1, 1) * x).unsqueeze(2) * Bh.unsqueeze(1)
        ssm_state.copy_(st.to(ssm_state.dtype))
        y = (st * Ch.unsqueeze(1)).sum(dim=2) + D.float().view(-1, 1) * x
        y = y.reshape(I) * f(gate)
        y = y * torch.rsqrt(y.pow(2).mean() + eps) * norm_w.float()
        out[t] = y
    return out


# ---- sampling helpers --------------------------------------------------------------------------------------------------
def log_softmax_at(logits: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    lf = logits.float()
    return lf.gather(-1, idx) - torch.logsumexp(lf, dim=-1, keepdim=True)
