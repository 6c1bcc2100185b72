"""Decode-step profile of a benchmark shape without paying for a prefill.

Builds the random-weight model, parks ``--batch`` sequences at context ``--ctx`` (KV pages allocated, contents zero — only
the timing matters), replays the last prompt token once (the full-prefix-hit path) and then runs ``--steps`` eager decode
steps with the stage profiler on. Prints the per-stage device times; run it under
``ncu --metrics gpu__time_duration.sum --clock-control none`` for a per-kernel launch list.
"""
from __future__ import annotations

import argparse
import json

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="qwen3-4b")
    ap.add_argument("--quant", default="jq4")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small captures)")
    ap.add_argument("--graphs", action="store_true")
    ap.add_argument("--prefill", action="store_true", help="profile the prefill of --batch prompts of --ctx tokens instead of decode steps")
    a = ap.parse_args()
    from deliverance_b200 import ops
    from deliverance_b200.ckpt.synthetic import SHAPES, SyntheticLoader
    from deliverance_b200.config import parse_config
    from deliverance_b200.engine.engine import Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.params import GeneratorParameters
    from deliverance_b200.utils.profiler import InferenceProfiler

    dev = torch.device("cuda", 0)
    shape = dict(SHAPES[a.shape])
    if a.layers:
        shape["num_hidden_layers"] = a.layers
    cfg = parse_config(shape)
    model = DecoderModel(cfg, dev, torch.bfloat16).load(SyntheticLoader(shape, 0, a.quant == "jq4", dev), head_quant="Q4" if a.quant == "jq4" else None)
    pages = (a.ctx + a.steps + 64) // 32 + 1
    conf = EngineConfig(max_seqs=a.batch, num_pages=a.batch * pages + 8, cuda_graphs=a.graphs)
    conf.kv.enabled = False
    eng = Engine(model, conf, eos_ids=(-1,))
    g = torch.Generator().manual_seed(0)
    for i in range(a.batch):
        r = eng.add_request(torch.randint(0, cfg.vocab_size, (a.ctx,), generator=g).tolist(), GeneratorParameters(max_tokens=1) if a.prefill else GeneratorParameters())
    if a.prefill:
        # one warm-up prefill of the same prompts (kernel attributes, scratch), then the measured one with the stage profiler on
        torch.cuda.synchronize()
        for timed in (False, True):
            if timed:
                for i in range(a.batch):
                    eng.add_request(torch.randint(0, cfg.vocab_size, (a.ctx,), generator=g).tolist(), GeneratorParameters(max_tokens=1))
            prof = InferenceProfiler(dev)
            model.profiler = prof if timed else None
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            steps = 0
            while eng.waiting or any(r.computed < len(r.fill) for r in eng.running):
                eng.step()
                steps += 1
            e1.record()
            torch.cuda.synchronize()
            ops.check_status(0)
            while eng.running or eng.waiting:  # let the requests finish (one more token each)
                eng.step()
            if timed:
                ms = e0.elapsed_time(e1)
                print(json.dumps({"shape": a.shape, "batch": a.batch, "prompt": a.ctx, "prefill_ms": ms, "engine_steps": steps,
                                  "tokens_per_s": a.batch * a.ctx / ms * 1e3}))
                prof.print_summary()
        return 0
    while eng.waiting and eng._admit(eng.waiting[0]):
        eng.waiting.pop(0)
    for r in eng.running:
        eng.kv.ensure_pages(r.pages, a.ctx)
        r.computed = a.ctx - 1  # as after a full prefix-cache hit: only the last prompt token is replayed
    eng.step()
    eng.step()
    torch.cuda.synchronize()
    prof = InferenceProfiler(dev)
    model.profiler = None if a.graphs else prof
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.step()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status(0)
    print(json.dumps({"shape": a.shape, "batch": a.batch, "ctx": a.ctx, "ms_per_step": e0.elapsed_time(e1) / a.steps}))
    if not a.graphs:
        prof.print_summary()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
