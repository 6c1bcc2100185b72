"""Roofline arithmetic for one decode step (or one prefill) of a decoder shape.

    python -m deliverance_b200.bench.roofline --shape qwen3-4b --quant jq4 --batch 64 --ctx 2048 [--tp 8] [--ms 5.93]

The target time of a step is the slowest of three streams that can overlap perfectly in the ideal kernel schedule:

* HBM: every weight byte is read once per step (JQ4: 0.5 byte per element + one fp32 scale per 32 elements; bf16: 2 bytes),
  the K/V rows of every cached token of every sequence are read once, the new rows are written;
* tensor cores: 2 x tokens x weight elements (+ attention QK^T and PV);
* NVLink (tensor parallel): the partial sums of the two row-parallel projections of every layer cross the links once in each
  direction per rank (one-shot all-reduce: every rank sends its [tokens, hidden] bf16 partial to size - 1 peers).

Denominators are the measured copy bandwidth and cuBLAS bf16 rate of this pool (``MEASURED_PEAKS.json`` at the repository root,
written by the test driver) or, when that file is absent, an earlier measurement of the same pool (6.65 TB/s, 1.59 PFLOP/s);
NVLink uses the measured peer-copy rate of 770 GB/s per direction. ``fraction`` = target time / measured time.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass
from typing import Optional

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS = 770.0  # measured peer copy, per direction per GPU


def load_peaks(path: Optional[str] = None) -> tuple:
    """(peaks dict, "measured" | "fallback")."""
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        if d.get("hbm_gbs") and d.get("bf16_tflops"):
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"])}, "measured"
    except (OSError, ValueError):
        pass
    return dict(FALLBACK), "fallback"


@dataclass
class StepCost:
    weight_bytes: float
    kv_bytes: float
    flops: float
    nvlink_bytes: float  # per rank, per direction

    @property
    def hbm_bytes(self) -> float:
        return self.weight_bytes + self.kv_bytes


def _weight_elems(cfg, tp: int) -> tuple:
    """(sharded matrix elements per rank, replicated elements per rank incl. the output head slice)."""
    h, L = cfg.hidden_size, cfg.num_layers
    q, kv = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    attn = h * (q + 2 * kv) + q * h
    if cfg.num_experts > 0:
        inter = cfg.moe_intermediate_size or cfg.intermediate_size
        ff_all = cfg.num_experts * 3 * h * inter
        ff_active = cfg.experts_per_token * 3 * h * inter
        router = h * cfg.num_experts
    else:
        ff_all = ff_active = 3 * h * cfg.intermediate_size
        router = 0
    head = cfg.vocab_size * h
    return L * (attn + ff_all) / tp, L * (attn + ff_active) / tp, L * router, head / tp


def decode_step_cost(cfg, batch: int, ctx: int, quant: str = "jq4", tp: int = 1, head_quant: Optional[str] = None) -> StepCost:
    """Algorithmic cost of one decode step of ``batch`` sequences with ``ctx`` cached tokens each, per rank."""
    stored, active, router, head = _weight_elems(cfg, tp)
    bpe = 0.5 + 4.0 / 32.0 if quant == "jq4" else 2.0
    head_bpe = 0.5 + 4.0 / 32.0 if (head_quant or ("q4" if quant == "jq4" else "")).lower() == "q4" else 2.0
    # MoE decode touches min(all experts, batch x k) experts per layer; dense models touch everything
    if cfg.num_experts > 0:
        inter = cfg.moe_intermediate_size or cfg.intermediate_size
        touched = min(cfg.num_experts, batch * cfg.experts_per_token) * 3 * cfg.hidden_size * inter / tp
        attn = stored - cfg.num_layers * cfg.num_experts * 3 * cfg.hidden_size * inter / tp
        weights = attn + cfg.num_layers * touched
    else:
        weights = stored
    weight_bytes = weights * bpe + router * 2.0 + head * head_bpe
    kv_heads = max(1.0, cfg.num_kv_heads / tp)
    n_attn = sum(1 for i in range(cfg.num_layers) if cfg.layer_type(i) != "mamba")
    row = 2 * kv_heads * cfg.head_dim * 2.0  # K and V, bf16
    seen = sum(min(ctx, cfg.window(i)) if cfg.window(i) else ctx for i in range(cfg.num_layers) if cfg.layer_type(i) != "mamba")
    kv_bytes = batch * (seen * row + n_attn * row)
    flops = 2.0 * batch * (active + router + head) + 4.0 * batch * seen * (cfg.num_heads / tp) * cfg.head_dim
    nv = 0.0
    if tp > 1:
        nv = 2 * n_attn * batch * cfg.hidden_size * 2.0 * (tp - 1)  # two row-parallel sums per layer, bf16 partials to every peer
    return StepCost(weight_bytes, kv_bytes, flops, nv)


def prefill_cost(cfg, batch: int, prompt: int, quant: str = "jq4", tp: int = 1) -> StepCost:
    """Algorithmic cost of prefilling ``batch`` prompts of ``prompt`` tokens, per rank: every matrix multiplies every token
    (the output head only the last token of each prompt), causal attention does half of the P x P score and value products.
    Weights are counted once (they are re-read per chunk in practice; the phase is tensor-bound at these sizes)."""
    stored, active, router, head = _weight_elems(cfg, tp)
    bpe = 0.5 + 4.0 / 32.0 if quant == "jq4" else 2.0
    tokens = batch * prompt
    attn_layers = [i for i in range(cfg.num_layers) if cfg.layer_type(i) != "mamba"]
    pairs = 0.0  # (query, key) pairs per sequence and layer
    for i in attn_layers:
        w = cfg.window(i)
        pairs += prompt * (prompt + 1) / 2.0 if not w or w >= prompt else w * (prompt - w) + w * (w + 1) / 2.0
    flops = 2.0 * tokens * (active + router) + 2.0 * batch * head + 4.0 * batch * pairs * (cfg.num_heads / tp) * cfg.head_dim
    kv_bytes = tokens * len(attn_layers) * 2 * max(1.0, cfg.num_kv_heads / tp) * cfg.head_dim * 2.0  # written once
    nv = 2 * len(attn_layers) * tokens * cfg.hidden_size * 2.0 * 2.0 * (tp - 1) / tp if tp > 1 else 0.0  # two-shot sums
    return StepCost(stored * bpe + router * 2.0 + head * bpe, kv_bytes, flops, nv)


def target_ms(cost: StepCost, peaks: dict, sustained: bool = True) -> dict:
    tf = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    t_hbm = cost.hbm_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
    t_mma = cost.flops / (tf * 1e12) * 1e3
    t_nv = cost.nvlink_bytes / (NVLINK_GBS * 1e9) * 1e3
    bound = max((t_hbm, "hbm"), (t_mma, "tensor"), (t_nv, "nvlink"))
    return {"hbm_ms": t_hbm, "tensor_ms": t_mma, "nvlink_ms": t_nv, "target_ms": bound[0], "bound": bound[1]}


def report(cfg, batch: int, ctx: int, quant: str, tp: int, measured_ms: Optional[float] = None, peaks_path: Optional[str] = None) -> dict:
    peaks, source = load_peaks(peaks_path)
    cost = decode_step_cost(cfg, batch, ctx, quant, tp)
    out = {"weight_gb": cost.weight_bytes / 1e9, "kv_gb": cost.kv_bytes / 1e9, "gflop": cost.flops / 1e9, "nvlink_mb": cost.nvlink_bytes / 1e6,
           **target_ms(cost, peaks), "denominators": f"of {source}", "peaks": peaks}
    if measured_ms:
        out["measured_ms"] = measured_ms
        out["fraction"] = out["target_ms"] / measured_ms
    return out


def prefill_report(cfg, batch: int, prompt: int, quant: str, tp: int, measured_ms: Optional[float] = None, peaks_path: Optional[str] = None) -> dict:
    peaks, source = load_peaks(peaks_path)
    cost = prefill_cost(cfg, batch, prompt, quant, tp)
    out = {"gflop": cost.flops / 1e9, "nvlink_mb": cost.nvlink_bytes / 1e6, **target_ms(cost, peaks), "denominators": f"of {source}"}
    if measured_ms:
        out["measured_ms"] = measured_ms
        out["fraction"] = out["target_ms"] / measured_ms
    return out


def main() -> int:
    from deliverance_b200.ckpt.synthetic import SHAPES
    from deliverance_b200.config import parse_config

    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="qwen3-4b", choices=sorted(SHAPES))
    ap.add_argument("--quant", default="jq4", choices=["jq4", "bf16"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ms", type=float, default=None, help="measured milliseconds per step")
    ap.add_argument("--peaks", default=None)
    ap.add_argument("--prefill", action="store_true", help="cost of prefilling --batch prompts of --ctx tokens instead of one decode step")
    a = ap.parse_args()
    if a.prefill:
        print(json.dumps(prefill_report(parse_config(dict(SHAPES[a.shape])), a.batch, a.ctx, a.quant, a.tp, a.ms, a.peaks), indent=1))
        return 0
    print(json.dumps(report(parse_config(dict(SHAPES[a.shape])), a.batch, a.ctx, a.quant, a.tp, a.ms, a.peaks), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
