"""PyTorch + cuBLAS + NCCL baseline of the headline benchmark: same architecture, same shapes, library kernels only.

A decoder (RMSNorm, q/k norm, RoPE, GQA, SwiGLU, tied head) written with ``torch.nn.functional`` calls: bf16 weights
through cuBLAS, attention through ``scaled_dot_product_attention`` over a contiguous static KV cache, tensor parallelism
by ``torch.distributed.all_reduce`` (NCCL) after ``o_proj`` and ``down_proj``. Mixture-of-experts shapes: softmax router, top-k,
renormalised weights; the routed rows are laid out per expert in a fixed-capacity buffer (4 x the average load, at least 8 rows;
rows beyond the capacity are dropped: a timing baseline, not an oracle) and every local expert runs as one batched cuBLAS GEMM
(``torch.bmm``), which keeps the step capturable; experts are split over the ranks when their number divides (tokens replicated,
outputs summed with an NCCL all-reduce), otherwise their inner dimension is. The decode step is captured in a CUDA graph
so the comparison is kernel against kernel, not launch overhead against launch overhead. None of this package's kernels
run here; ``bench.py --impl torch`` prints its numbers in the same JSON form as the framework's own arm.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


class TorchDecoder:
    def __init__(self, shape: dict, device, rank: int = 0, world: int = 1, seed: int = 0, max_batch: int = 64, max_ctx: int = 4096):
        self.dev, self.rank, self.world = device, rank, world
        H, L = shape["hidden_size"], shape["num_hidden_layers"]
        self.nh, self.nkv, self.hd = shape["num_attention_heads"] // world, max(1, shape["num_key_value_heads"] // world), shape.get("head_dim") or shape["hidden_size"] // shape["num_attention_heads"]
        I = shape["intermediate_size"] // world
        self.E = int(shape.get("num_local_experts") or shape.get("num_experts") or 0)
        self.topk = int(shape.get("num_experts_per_tok") or 0)
        self.ep = self.E > 0 and self.E % world == 0
        self.e_loc = (self.E // world) if self.ep else self.E
        self.e0 = rank * self.e_loc if self.ep else 0
        Im = int(shape.get("moe_intermediate_size") or shape["intermediate_size"])
        self.Im = Im if self.ep else Im // world
        self.eps, self.V, self.H, self.L = shape.get("rms_norm_eps", 1e-6), shape["vocab_size"], H, L
        g = torch.Generator(device=device).manual_seed(seed + 17 * rank)
        w = lambda *s: (torch.randn(*s, device=device, dtype=torch.float32, generator=g) * 0.02).to(torch.bfloat16)  # noqa: E731
        one = lambda n: torch.ones(n, device=device, dtype=torch.bfloat16)  # noqa: E731
        self.embed = w(self.V, H)
        if self.E:
            self.layers = [dict(n1=one(H), qkv=w((self.nh + 2 * self.nkv) * self.hd, H), qn=one(self.hd), kn=one(self.hd), o=w(H, self.nh * self.hd),
                                n2=one(H), router=w(self.E, H), egu=w(self.e_loc, H, 2 * self.Im), edown=w(self.e_loc, self.Im, H)) for _ in range(L)]
        else:
            self.layers = [dict(n1=one(H), qkv=w((self.nh + 2 * self.nkv) * self.hd, H), qn=one(self.hd), kn=one(self.hd), o=w(H, self.nh * self.hd),
                                n2=one(H), gu=w(2 * I, H), down=w(H, I)) for _ in range(L)]
        self.norm = one(H)
        inv = 1.0 / (shape.get("rope_theta", 1e6) ** (torch.arange(0, self.hd, 2, device=device, dtype=torch.float32) / self.hd))
        ang = torch.arange(max_ctx, device=device, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.k = [torch.zeros(max_batch, self.nkv, max_ctx, self.hd, device=device, dtype=torch.bfloat16) for _ in range(L)]
        self.v = [torch.zeros_like(t) for t in self.k]
        self.max_ctx = max_ctx

    def _rope(self, x, pos):  # x [B, T, h, d], pos [B, T]
        c, s = self.cos[pos][:, :, None, :], self.sin[pos][:, :, None, :]
        x1, x2 = x[..., : self.hd // 2].float(), x[..., self.hd // 2 :].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)

    def _reduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t)
        return t

    def _moe(self, h, lw):
        """h ``[N, H]`` -> routed expert output ``[N, H]`` (before the sum over ranks)."""
        N, E, k, C_e = h.shape[0], self.E, self.topk, self.e_loc
        cap = max(8, 4 * ((N * k + E - 1) // E))
        probs = torch.softmax(F.linear(h, lw["router"]).float(), dim=-1)
        wgt, idx = torch.topk(probs, k, dim=-1)
        wgt = (wgt / wgt.sum(-1, keepdim=True)).to(h.dtype).flatten()
        flat_e = idx.flatten()
        order = torch.argsort(flat_e, stable=True)
        sorted_e = flat_e[order]
        counts = torch.zeros(E, dtype=flat_e.dtype, device=h.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))  # (bincount syncs)
        starts = torch.cumsum(counts, 0) - counts
        within = torch.arange(N * k, device=h.device) - starts[sorted_e]
        local = sorted_e - self.e0
        keep = (within < cap) & (local >= 0) & (local < C_e)
        slot = torch.where(keep, local * cap + within, torch.full_like(within, C_e * cap))  # dropped rows go to a dummy slot
        token = order // k
        xp = torch.zeros(C_e * cap + 1, self.H, device=h.device, dtype=h.dtype)
        xp.index_copy_(0, slot, h[token])
        gu = torch.bmm(xp[:-1].view(C_e, cap, self.H), lw["egu"])
        g, u = gu.chunk(2, -1)
        y = torch.bmm(F.silu(g) * u, lw["edown"]).view(C_e * cap, self.H)
        y = torch.cat([y, torch.zeros(1, self.H, device=h.device, dtype=h.dtype)], 0)
        rows = y[slot] * (wgt[order] * keep.to(h.dtype))[:, None]
        return torch.zeros(N, self.H, device=h.device, dtype=h.dtype).index_add_(0, token, rows)

    def forward(self, ids, pos, mask):
        """ids, pos ``[B, T]``; mask ``[B, 1, T, max_ctx]`` additive (``None`` = causal prefill from position 0); writes K/V at
        ``pos`` and returns last-token logits."""
        B, T = ids.shape
        x = self.embed[ids]
        bidx = torch.arange(B, device=self.dev)[:, None].expand(B, T)
        for i, lw in enumerate(self.layers):
            h = F.rms_norm(x, (self.H,), lw["n1"], self.eps)
            qkv = F.linear(h, lw["qkv"]).view(B, T, self.nh + 2 * self.nkv, self.hd)
            q, k, v = qkv[:, :, : self.nh], qkv[:, :, self.nh : self.nh + self.nkv], qkv[:, :, self.nh + self.nkv :]
            q = self._rope(F.rms_norm(q, (self.hd,), lw["qn"], self.eps), pos)
            k = self._rope(F.rms_norm(k, (self.hd,), lw["kn"], self.eps), pos)
            self.k[i][bidx, :, pos] = k
            self.v[i][bidx, :, pos] = v
            if mask is None:  # prefill from position 0: plain causal attention over the T new keys (flash backend)
                a = F.scaled_dot_product_attention(q.transpose(1, 2), self.k[i][:B, :, :T], self.v[i][:B, :, :T], is_causal=True, enable_gqa=True)
            else:
                a = F.scaled_dot_product_attention(q.transpose(1, 2), self.k[i][:B], self.v[i][:B], attn_mask=mask, enable_gqa=True)
            x = x + self._reduce(F.linear(a.transpose(1, 2).reshape(B, T, -1), lw["o"]))
            h = F.rms_norm(x, (self.H,), lw["n2"], self.eps)
            if self.E:
                x = x + self._reduce(self._moe(h.reshape(B * T, self.H), lw)).view(B, T, self.H)
            else:
                gu = F.linear(h, lw["gu"])
                g, u = gu.chunk(2, -1)
                x = x + self._reduce(F.linear(F.silu(g) * u, lw["down"]))
        x = F.rms_norm(x[:, -1], (self.H,), self.norm, self.eps)
        return F.linear(x, self.embed)


def run(args, dev, rank: int, world: int, shape: dict, sync_all, max_over_ranks) -> dict:
    """Prefill ``prompt_len`` tokens for ``batch`` sequences, then time ``steps`` graph-replayed greedy decode steps."""
    B, P = args.batch, args.prompt_len
    ctx = ((P + args.warmup + args.steps + 64 + 127) // 128) * 128
    m = TorchDecoder(shape, dev, rank, world, max_batch=B, max_ctx=ctx)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, m.V, (B, P), generator=g).to(dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kpos = torch.arange(ctx, device=dev)
    sync_all()
    ev0.record()
    nxt = []
    with torch.no_grad():
        for b0 in range(0, B, 4):  # 4 sequences (8192 tokens) per prefill batch, like the framework's token budget
            ids = prompts[b0 : b0 + 4]
            pos = torch.arange(P, device=dev)[None].expand(ids.shape[0], P)
            sub = TorchDecoderView(m, b0, ids.shape[0])
            nxt.append(sub.forward(ids, pos, None).argmax(-1))
    ev1.record()
    sync_all()
    prefill_ms = max_over_ranks(ev0.elapsed_time(ev1))
    tok = torch.cat(nxt)[:, None].contiguous()
    pos = torch.full((B, 1), P, device=dev, dtype=torch.long)
    mask = torch.zeros(B, 1, 1, ctx, device=dev, dtype=torch.bfloat16)

    def step():
        mask.copy_(torch.where(kpos[None, None, None, :] <= pos[:, None, :, None], 0.0, float("-inf")))
        logits = m.forward(tok, pos, mask)
        tok.copy_(logits.argmax(-1, keepdim=True))
        pos.add_(1)

    with torch.no_grad():
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for _ in range(args.warmup):
            graph.replay()
        sync_all()
        ev0.record()
        for _ in range(args.steps):
            graph.replay()
        ev1.record()
        sync_all()
    ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
    return {"ms_per_step": ms, "decode_tok_s": B / (ms / 1e3), "prefill_ms": prefill_ms, "prefill_tok_s": B * P / (prefill_ms / 1e3)}


class TorchDecoderView:
    """Runs a slice ``[b0, b0+n)`` of the static KV cache through the same weights (prefill in sub-batches)."""

    def __init__(self, m: TorchDecoder, b0: int, n: int):
        self.m, self.b0, self.n = m, b0, n

    def forward(self, ids, pos, mask):
        m = self.m
        k, v = m.k, m.v
        m.k, m.v = [t[self.b0 : self.b0 + self.n] for t in k], [t[self.b0 : self.b0 + self.n] for t in v]
        try:
            return m.forward(ids, pos, mask)
        finally:
            m.k, m.v = k, v
