"""Prefill attention micro-benchmark: the tcgen05 / TMA kernel against the mma.sync kernel (and torch's fused SDPA as a library
yardstick) on ragged causal prefill over the paged cache.

Every case holds ``--seqs`` sequences of ``--len`` new tokens each (no cached prefix), Qwen3-4B heads by default (32 query heads,
8 KV heads, head_dim 128). Time is taken with CUDA events after warm-up; the FLOP count is the causal half of 4 * T * ctx * H * D.
Prints one JSON line per case with the fraction of the measured cuBLAS bf16 rate (``MEASURED_PEAKS.json`` when present).
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from .gemm_bench import peaks


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="1x2048,8x2048,2x8192", help="comma list of <sequences>x<tokens>")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--impls", default="tc,mma,sdpa")
    a = ap.parse_args()
    from deliverance_b200 import ops

    dev = torch.device("cuda", 0)
    _, tf, src = peaks()
    H, KV, D, page = a.heads, a.kv_heads, a.head_dim, a.page
    scale = 1.0 / math.sqrt(D)
    for case in a.cases.split(","):
        S, L = (int(v) for v in case.split("x"))
        T = S * L
        pages_per = (L + page - 1) // page
        n_pages = S * pages_per + 1
        kc = (torch.randn(n_pages, KV, page, D, device=dev) * 0.5).to(torch.bfloat16)
        vc = (torch.randn(n_pages, KV, page, D, device=dev) * 0.5).to(torch.bfloat16)
        bt = (torch.randperm(n_pages - 1, device=dev) + 1).to(torch.int32).reshape(S, pages_per)
        q = (torch.randn(T, H * D, device=dev) * 0.5).to(torch.bfloat16)
        ql = torch.full((S,), L, dtype=torch.int32, device=dev)
        qs = (torch.arange(S, device=dev, dtype=torch.int32) * L)
        lens = [L] * S
        flops = 4.0 * H * D * S * (L * (L + 1) / 2)
        outs = {}
        for impl in a.impls.split(","):
            if impl == "sdpa":
                # dense [S, H, L, D] views of the same values (the copy out of the pages is not timed)
                kd = kc[bt.long()].permute(0, 2, 1, 3, 4).reshape(S, KV, pages_per * page, D)[:, :, :L]
                vd = vc[bt.long()].permute(0, 2, 1, 3, 4).reshape(S, KV, pages_per * page, D)[:, :, :L]
                qd = q.reshape(S, L, H, D).permute(0, 2, 1, 3)
                fn = lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, is_causal=True, scale=scale, enable_gqa=True)  # noqa: E731
            else:
                fn = lambda impl=impl: ops.prefill_attention(q, kc, vc, bt, qs, ql, ql, H, scale, 0.0, 0, True, impl=impl, q_len_host=lens)  # noqa: E731
            for _ in range(3):
                o = fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                o = fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / a.iters
            outs[impl] = o.permute(0, 2, 1, 3).reshape(T, H * D) if impl == "sdpa" else o
            row = {"case": case, "impl": impl, "H": H, "KV": KV, "D": D, "us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                   "frac_bf16": round(flops / us / 1e6 / tf, 3), "peaks": src}
            if impl != a.impls.split(",")[0]:
                first = outs[a.impls.split(",")[0]].float()
                row["rel_vs_first"] = round(float((outs[impl].float() - first).norm() / first.norm()), 5)
            print(json.dumps(row), flush=True)
        ops.check_status(0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
