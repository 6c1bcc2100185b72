"""Single-request inference benchmark with the reference's CSV columns.

The reference's ``InferenceBenchmark`` CLI (core/.../benchmark/InferenceBenchmark.java:67,1037-1072; metric definitions in
core/InferenceBenchmark.md:92-98) runs a list of prompts one at a time and writes a CSV with, per prompt, the prompt and
generated token counts, total and generation time and ``tokens_per_second`` = generated tokens after the first divided by
(total - time to first token). This tool does the same through the public API:

    python -m deliverance_b200.bench.inference_benchmark --model DIR [--prompts FILE] [--max-tokens 256] [--out FILE.csv]
        [--output-head-quantization Q4] [--quantize-on-demand] [--runs 1] [--profile-stages]

Prompts: one per line in ``--prompts`` (default: five built-in prompts). ``--synthetic SHAPE`` benchmarks a random-init
model of a named shape instead of a directory (token-id prompts of ``--prompt-len`` random ids).
"""
from __future__ import annotations

import argparse
import csv
import sys
import time

DEFAULT_PROMPTS = [
    "Explain why the sky is blue in three sentences.",
    "Write a short poem about autumn rain.",
    "List five uses of a paperclip.",
    "Summarise the plot of Romeo and Juliet.",
    "What is the capital of Australia, and what is it known for?",
]
COLUMNS = ["run", "prompt_index", "prompt_tokens", "generated_tokens", "ttft_ms", "generation_ms", "total_ms", "tokens_per_second", "finish_reason"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--synthetic", help="shape name from ckpt.synthetic.SHAPES instead of a model directory")
    ap.add_argument("--quant", default="jq4", choices=["jq4", "bf16"])
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--prompts")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--runs", type=int, default=1)
    ap.add_argument("--out", default="-")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--output-head-quantization", default=None)
    ap.add_argument("--quantize-on-demand", action="store_true")
    ap.add_argument("--profile-stages", action="store_true")
    ap.add_argument("--temperature", type=float, default=0.0)
    a = ap.parse_args()
    import torch

    from deliverance_b200.params import GeneratorParameters

    if a.synthetic:
        from deliverance_b200.ckpt.synthetic import SHAPES, SyntheticLoader
        from deliverance_b200.config import parse_config
        from deliverance_b200.engine.engine import Engine, EngineConfig
        from deliverance_b200.models.transformer import DecoderModel

        dev = torch.device("cuda" if torch.cuda.is_available() and a.device != "cpu" else "cpu")
        shape = SHAPES[a.synthetic]
        cfg = parse_config(dict(shape))
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        model = DecoderModel(cfg, dev, dtype).load(SyntheticLoader(shape, 0, a.quant == "jq4", dev, dtype=dtype),
                                                   head_quant="Q4" if a.quant == "jq4" else None)
        eng = Engine(model, EngineConfig(max_seqs=1, num_pages=(a.prompt_len + a.max_tokens) // 32 + 8), eos_ids=(-1,))
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(5)]

        def run_one(p):
            r = eng.generate(p, GeneratorParameters(max_tokens=a.max_tokens, temperature=a.temperature))
            return r
    else:
        if not a.model:
            ap.error("--model or --synthetic is required")
        from deliverance_b200.api import AutoModelForCausalLM

        b = AutoModelForCausalLM.new_builder(a.model).with_device(a.device).with_output_head_quantization(a.output_head_quantization)
        b = b.with_quantize_on_demand(a.quantize_on_demand).with_profile_stages(a.profile_stages)
        clm = b.build()
        if a.prompts:
            with open(a.prompts) as f:
                prompts = [l.rstrip("\n") for l in f if l.strip()]
        else:
            prompts = DEFAULT_PROMPTS

        def run_one(p):
            text = clm.prompt_builder().add_user(p).build() if clm.tokenizer.chat_template else p
            return clm.generate(text, GeneratorParameters(max_tokens=a.max_tokens, temperature=a.temperature))
    fh = sys.stdout if a.out == "-" else open(a.out, "w", newline="")
    w = csv.writer(fh)
    w.writerow(COLUMNS)
    for run in range(a.runs):
        for i, p in enumerate(prompts):
            t0 = time.perf_counter()
            r = run_one(p)
            total = (time.perf_counter() - t0) * 1e3
            ttft = getattr(r, "ttft_ms", None) or 0.0
            gen_ms = max(total - ttft, 1e-9)
            n = r.generated_tokens
            tps = (n - 1) / (gen_ms / 1e3) if n > 1 else 0.0
            w.writerow([run, i, r.prompt_tokens, n, f"{ttft:.2f}", f"{gen_ms:.2f}", f"{total:.2f}", f"{tps:.2f}", r.finish_reason.wire])
            fh.flush()
    if not a.synthetic and a.profile_stages and getattr(clm.model, "profiler", None) is not None:
        print(clm.model.profiler.summary(), file=sys.stderr)
    if fh is not sys.stdout:
        fh.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
