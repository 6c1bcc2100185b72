"""Decode-chain micro-benchmark: one persistent launch per layer against the same steps as separate kernels.

Builds ``--layers`` independent sets of JQ4 weights of the given shape (together larger than the 126 MB L2, so every layer streams
its weights from HBM), captures both variants of the per-layer sequence
``o_proj -> add + norm -> gate|up -> act * up -> down -> add + norm -> q|k|v -> q/k norm + rotary + KV write`` for all layers in a
CUDA graph each, and times graph replays with CUDA events. Prints one JSON line per token count with microseconds per layer, the
weight bandwidth and its fraction of the measured copy bandwidth (``MEASURED_PEAKS.json`` when present).
"""
from __future__ import annotations

import argparse
import json

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", default="1,8,64")
    ap.add_argument("--hidden", type=int, default=2560)
    ap.add_argument("--inter", type=int, default=9728)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="", help="chain | separate: build and time one variant only (small profiler captures)")
    a = ap.parse_args()
    from deliverance_b200 import ops
    from deliverance_b200.bench.gemm_bench import peaks
    from deliverance_b200.ckpt.safetensors_io import Q4Tensor
    from deliverance_b200.ops import LinearWeight, ref

    dev = torch.device("cuda", 0)
    e = ops.require_ext()
    hbm, _, src = peaks()
    H, KV, D, hid, I = a.heads, a.kv_heads, a.head_dim, a.hidden, a.inter
    R, page = 64, 32

    def lin(N, K):
        w = torch.randn(N, K, device=dev) * 0.02
        p, s = ops.q4_quantize(w)
        return LinearWeight(Q4Tensor(p, s, (N, K))).to(dev)

    layers = []
    for _ in range(a.layers):
        layers.append({"o": lin(hid, H * D), "gu": lin(2 * I, hid), "dn": lin(hid, I), "qkv": lin((H + 2 * KV) * D, hid),
                       "n1": torch.ones(hid, dtype=torch.bfloat16, device=dev), "n2": torch.ones(hid, dtype=torch.bfloat16, device=dev),
                       "qn": torch.ones(D, dtype=torch.bfloat16, device=dev), "kn": torch.ones(D, dtype=torch.bfloat16, device=dev)})
    wbytes = sum(l[k].nbytes() for l in layers[:1] for k in ("o", "gu", "dn", "qkv"))
    cos, sin = ref.rope_tables(D, 4096, 1e6, 1.0)
    cos, sin = cos.to(dev), sin.to(dev)
    kc = torch.zeros(8, KV, page, D, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    attn = (torch.randn(R, H * D, device=dev) * 0.1).to(torch.bfloat16)
    res = (torch.randn(R, hid, device=dev) * 0.1).to(torch.bfloat16)
    bx1, bh, bx2, bq = (torch.zeros(R, n, dtype=torch.bfloat16, device=dev) for n in (hid, I, hid, H * D))
    chains = []
    for l in layers:
        ch = e.DecodeChain()
        ch.add_op(l["o"].handle(), attn, 1, residual=res, norm_w=l["n1"], out=bx1)
        ch.add_op(l["gu"].handle(), bx1, 2, dep=True, scale_src=0, out=bh)
        ch.add_op(l["dn"].handle(), bh, 1, dep=True, residual=res, norm_w=l["n2"], out=bx2)
        ch.add_op(l["qkv"].handle(), bx2, 3, dep=True, scale_src=2, out=bq)
        ch.set_qkv(l["qn"], l["kn"], cos, sin, kc, vc, H, KV, 1e-6, 0.0)
        chains.append(ch)
    for M in (int(v) for v in a.m.split(",")):
        pos = torch.arange(M, dtype=torch.int32, device=dev)
        slots = torch.arange(M, dtype=torch.int64, device=dev)

        def run_chain():
            for ch in chains:
                ch.run(M, pos, slots)

        def run_separate():
            r = res[:M]
            for l in layers:
                x1 = ops.add_rmsnorm(ops.linear(attn[:M], l["o"]), r, l["n1"], 1e-6)
                hh = ops.act_mul(ops.linear(x1, l["gu"]), "silu")
                x2 = ops.add_rmsnorm(ops.linear(hh, l["dn"]), r, l["n2"], 1e-6)
                ops.linear_rope_kv(x2, l["qkv"], pos, slots, l["qn"], l["kn"], cos, sin, kc, vc, H, KV, D, 1e-6, 0.0)

        row = {"M": M, "layers": a.layers, "weight_MB_per_layer": round(wbytes / 1e6, 1), "peaks": src}
        for name, fn in (("chain", run_chain), ("separate", run_separate)):
            if a.only and a.only != name:
                continue
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (a.iters * a.layers)
            row[f"{name}_us_per_layer"] = round(us, 2)
            row[f"{name}_frac_hbm"] = round(wbytes / us / 1e3 / hbm, 3)
        ops.check_status(0)
        print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
