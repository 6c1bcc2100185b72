"""Single-request inference benchmark with the reference's CSV columns.

The reference's ``InferenceBenchmark`` CLI (core/.../benchmark/InferenceBenchmark.java:67,1037-1072; metric definitions in
core/InferenceBenchmark.md:92-98) runs a list of prompts one at a time and writes a CSV with, per prompt, the prompt and
generated token counts, total and generation time and ``tokens_per_second`` = generated tokens after the first divided by
(total - time to first token). This tool does the same through the public API:

    python -m deliverance_b200.bench.inference_benchmark --model DIR [--questions FILE.jsonl] [--max-tokens 256] [--out FILE.csv]
        [--jsonl-output FILE.jsonl] [--config AUTO_MODEL_CONFIG.json] [--output-head-quantization Q4] [--quantize-on-demand]
        [--runs 1] [--profile-stages]

The CSV has the reference's columns (engine, model, case_id, category, turn, prompt_chars, prompt_tokens, generated_tokens,
total_ms, generation_ms, tokens_per_second, response_chars, finish_reason) plus ttft_ms; ``--jsonl-output`` writes one
transcript record per turn (messages so far, rendered prompt, response text, the same metrics), flushed after every turn.
Suites: the built-in multi-category set, or MT-Bench style questions (``--questions``; multi-turn cases continue the chat).
``--synthetic SHAPE`` benchmarks a random-init model of a named shape (token-id prompts of ``--prompt-len`` random ids).
"""
from __future__ import annotations

import argparse
import csv
import sys
import time

# built-in suite: (case_id, category, turns) in the shape of MT-Bench questions (the reference's default suite is an MT-Bench-derived subset)
DEFAULT_SUITE = [
    ("reasoning-1", "reasoning", ["Three friends split a bill of 90 dollars so that each pays twice the previous one. How much does each pay?",
                                  "Now explain the answer to a ten-year-old."]),
    ("math-1", "math", ["What is the sum of the first 20 odd numbers? Show the steps."]),
    ("coding-1", "coding", ["Write a Python function that checks whether a string is a palindrome, ignoring punctuation.",
                            "Add type hints and a docstring."]),
    ("extraction-1", "extraction", ["Extract the year, the city and the winner from: 'In 1998 the final in Paris was won by France.' Answer as JSON."]),
    ("stem-1", "stem", ["Explain why the sky is blue in three sentences."]),
    ("humanities-1", "humanities", ["Summarise the causes of the French Revolution in one paragraph."]),
    ("writing-1", "writing", ["Write a short poem about autumn rain."]),
]
COLUMNS = ["engine", "model", "case_id", "category", "turn", "prompt_chars", "prompt_tokens", "generated_tokens", "total_ms", "generation_ms",
           "tokens_per_second", "response_chars", "finish_reason", "ttft_ms"]


def load_suite(path):
    """MT-Bench style JSONL: one object per line with ``question_id``, ``category`` and ``turns`` (list of user messages);
    a line may carry ``guided_choice`` / ``guided_regex`` / ``guided_json`` (the reference's guided support suite), applied to
    every turn of the case."""
    import json

    suite = []
    with open(path) as f:
        for line in f:
            if line.strip():
                q = json.loads(line)
                guided = {k: q[k] for k in ("guided_choice", "guided_regex", "guided_json") if q.get(k) is not None}
                suite.append((str(q.get("question_id", len(suite))), q.get("category", ""), list(q["turns"]), guided))
    return suite


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--synthetic", help="shape name from ckpt.synthetic.SHAPES instead of a model directory")
    ap.add_argument("--quant", default="jq4", choices=["jq4", "bf16"])
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--questions", help="MT-Bench style JSONL (question_id, category, turns)")
    ap.add_argument("--jsonl-output")
    ap.add_argument("--config", help="AutoModelConfig JSON (this package's keys or the reference's layout)")
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
        from deliverance_b200.api import AutoModelConfig, AutoModelForCausalLM

        b = AutoModelForCausalLM.new_builder(a.model)
        if a.config:
            b = b.with_config(AutoModelConfig.from_json(a.config))
        b = b.with_device(a.device)
        if a.output_head_quantization:
            b = b.with_output_head_quantization(a.output_head_quantization)
        b = b.with_quantize_on_demand(a.quantize_on_demand or b.conf.quantize_on_demand).with_profile_stages(a.profile_stages)
        clm = b.build()
    fh = sys.stdout if a.out == "-" else open(a.out, "w", newline="")
    jl = open(a.jsonl_output, "w") if a.jsonl_output else None
    w = csv.writer(fh)
    w.writerow(COLUMNS)

    def record(case_id, category, turn, prompt_chars, r, total, extra=None):
        ttft = getattr(r, "ttft_ms", None) or 0.0
        gen_ms = max(total - ttft, 1e-9)
        n = r.generated_tokens
        tps = (n - 1) / (gen_ms / 1e3) if n > 1 else 0.0
        row = ["deliverance_b200", a.synthetic or clm.name, case_id, category, turn, prompt_chars, r.prompt_tokens, n, f"{total:.2f}", f"{gen_ms:.2f}",
               f"{tps:.2f}", len(r.text or ""), r.finish_reason.wire, f"{ttft:.2f}"]
        w.writerow(row)
        fh.flush()
        if jl is not None:
            import json

            jl.write(json.dumps({**dict(zip(COLUMNS, row)), **(extra or {})}) + "\n")
            jl.flush()

    for run in range(a.runs):
        if a.synthetic:
            for i, p in enumerate(prompts):
                t0 = time.perf_counter()
                r = run_one(p)
                record(f"synthetic-{i}", "synthetic", 1, 0, r, (time.perf_counter() - t0) * 1e3)
            continue
        suite = load_suite(a.questions) if a.questions else DEFAULT_SUITE
        for case in suite:
            case_id, category, turns = case[:3]
            guided = case[3] if len(case) > 3 else {}
            messages = []
            for ti, user in enumerate(turns, 1):
                messages.append({"role": "user", "content": user})
                pb = clm.prompt_builder()
                for m in messages:
                    pb = pb.add_user(m["content"]) if m["role"] == "user" else pb.add_assistant(m["content"])
                ctx = pb.build()
                t0 = time.perf_counter()
                r = clm.generate(ctx, GeneratorParameters(max_tokens=a.max_tokens, temperature=a.temperature, **guided))
                total = (time.perf_counter() - t0) * 1e3
                record(case_id, category, ti, len(ctx.prompt), r, total,
                       {"messages": list(messages), "rendered_prompt": ctx.prompt, "response_text": r.text,
                        "response_text_with_special_tokens": r.text_with_special_tokens})
                messages.append({"role": "assistant", "content": r.text})
    if jl is not None:
        jl.close()
    if not a.synthetic and a.profile_stages and getattr(clm.model, "profiler", None) is not None:
        print(clm.model.profiler.summary(), file=sys.stderr)
    if fh is not sys.stdout:
        fh.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
