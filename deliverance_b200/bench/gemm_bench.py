"""GEMM micro-benchmark: achieved weight bandwidth / FLOP rate of ``ops.linear`` for the decode and prefill shapes.

Each (N, K) shape gets enough distinct weight copies to exceed the 126 MB L2, launches cycle through them, and the time is
taken with CUDA events after warm-up. Prints one JSON line per case with the fraction of the measured HBM copy bandwidth
and of the measured cuBLAS bf16 rate (``MEASURED_PEAKS.json`` when present, else 6.65 TB/s / 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, "fallback"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", default="1,8,64,256,2048")
    ap.add_argument("--shapes", default="6144x2560,2560x4096,19456x2560,2560x9728")
    ap.add_argument("--quant", default="jq4")
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--impl", type=int, default=0)
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul on bf16 weights")
    ap.add_argument("--persist", default="off", choices=["off", "ordered", "race"],
                    help="prefill-size JQ4 shapes on the persistent kernel wherever it applies: issuers in k-block order or racing")
    a = ap.parse_args()
    from deliverance_b200 import ops
    from deliverance_b200.ckpt.safetensors_io import Q4Tensor
    from deliverance_b200.ops import LinearWeight

    dev = torch.device("cuda", 0)
    if a.persist != "off":
        ops.require_ext().gemm_persist(True, True, a.persist == "ordered")
    hbm, tf, src = peaks()
    for shp in a.shapes.split(","):
        N, K = (int(v) for v in shp.split("x"))
        per = N * K * (0.5625 if a.quant == "jq4" else 2)
        copies = max(2, int(300e6 // per) + 1)
        ws = []
        for c in range(copies):
            w = torch.randn(N, K, device=dev) * 0.02
            if a.quant == "jq4":
                p, s = ops.q4_quantize(w)
                ws.append(LinearWeight(Q4Tensor(p, s, (N, K))).to(dev))
            else:
                ws.append(LinearWeight(w.to(torch.bfloat16)))
        dense = [w.dense(torch.bfloat16) for w in ws] if a.cublas else None
        for M in (int(v) for v in a.m.split(",")):
            x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
            for i in range(copies):
                ops.linear(x, ws[i], impl=a.impl)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(a.iters):
                ops.linear(x, ws[i % copies], impl=a.impl)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / a.iters
            row = {"N": N, "K": K, "M": M, "quant": a.quant, "us": round(us, 2), "weight_GBs": round(per / us / 1e3, 1),
                   "frac_hbm": round(per / us / 1e3 / hbm, 3), "tflops": round(2.0 * M * N * K / us / 1e6, 1),
                   "frac_bf16": round(2.0 * M * N * K / us / 1e6 / tf, 3), "peaks": src}
            if a.cublas:
                for i in range(copies):
                    torch.matmul(x, dense[i].t())
                torch.cuda.synchronize()
                e0.record()
                for i in range(a.iters):
                    torch.matmul(x, dense[i % copies].t())
                e1.record()
                torch.cuda.synchronize()
                row["cublas_bf16_us"] = round(e0.elapsed_time(e1) * 1e3 / a.iters, 2)
            print(json.dumps(row), flush=True)
        ops.check_status(0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
