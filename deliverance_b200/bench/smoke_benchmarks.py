"""Two small single-model benchmark CLIs that ship example generations with their numbers.

    python -m deliverance_b200.bench.smoke_benchmarks thinking --model DIR [--enable-thinking] [--max-tokens 512] [--out FILE.jsonl]
    python -m deliverance_b200.bench.smoke_benchmarks lora --model DIR --adapter ADAPTER_DIR [--mode merge|hotswap] [--out FILE.csv]

``thinking``: a fixed list of short reasoning questions, each with a pass predicate over the text after the last ``final:``
marker (needles that must / must not occur, case-insensitive); multi-turn cases continue the chat; one JSONL row per case with
``timestamp, case_id, pass, finish_reason, generated_tokens, time_ms, time_to_first_token_ms, response`` and a summary line
``passed=P/N max_token_warnings=W`` (reference: core/.../benchmark/ThinkingSmokeBenchmark.java:42-150, cases :151-200,
answer extraction :205-252).

``lora``: the same prompts against the base model and against the model with a LoRA adapter (merged at load, or hot-swapped
at run time on one loaded model), CSV with the single-request benchmark's columns plus ``variant`` = ``base`` /
``lora-adapted`` so rows can be diffed across variants (reference: core/.../benchmark/LoraAdapterBenchmark.java:40-75).
"""
from __future__ import annotations

import argparse
import csv
import datetime
import json
import sys
import time
from dataclasses import dataclass, field
from typing import Optional

INSTRUCTION = " Think it through, then give the answer on a last line that starts with 'final:'."


@dataclass
class SmokeCase:
    id: str
    prompts: list
    must: list = field(default_factory=list)      # every needle occurs in the final answer
    must_not: list = field(default_factory=list)  # no needle occurs in the final answer
    any_of: list = field(default_factory=list)    # at least one occurs (when non-empty)

    def check(self, answer: str) -> bool:
        a = answer.lower()
        return (all(n.lower() in a for n in self.must) and not any(n.lower() in a for n in self.must_not)
                and (not self.any_of or any(n.lower() in a for n in self.any_of)))


CASES = [
    SmokeCase("square-area", ["A square has a perimeter of 36 cm. What is its area in square centimetres?" + INSTRUCTION], must=["81"]),
    SmokeCase("bat-ball", ["A bat and a ball cost 1.10 together and the bat costs 1.00 more than the ball. How much is the ball?" + INSTRUCTION],
              any_of=["0.05", "5 cents", "five cents"], must_not=["0.10", "10 cents"]),
    SmokeCase("calendar", ["If today is Wednesday, which day of the week is it 10 days from now?" + INSTRUCTION], must=["saturday"]),
    SmokeCase("odd-one-out", ["Which word does not belong: apple, banana, carrot, cherry?" + INSTRUCTION], must=["carrot"]),
    SmokeCase("syllogism", ["All bloops are razzies and all razzies are lazzies. Are all bloops lazzies? Answer yes or no." + INSTRUCTION],
              must=["yes"]),
    SmokeCase("missing-dollar", ["Three guests pay 30 for a room, get 5 back, the clerk keeps 2 and returns 1 to each. Each paid 9, 27 in total, "
                                 "plus 2 is 29. Is a dollar actually missing? Answer yes or no." + INSTRUCTION], must=["no"], must_not=["yes"]),
    SmokeCase("follow-up", ["What is 17 times 6?" + INSTRUCTION, "Now subtract 2 from that." + INSTRUCTION], must=["100"]),
]


def final_answer(text: str) -> str:
    """The part a pass predicate looks at: reasoning blocks and back-ticks removed, everything after the last ``final:``."""
    import re

    t = re.sub(r"<think>.*?</think>", "", text or "", flags=re.S)
    t = t.replace("<think>", "").replace("</think>", "").replace("`", "")
    i = t.lower().rfind("final:")
    return (t[i + 6:] if i >= 0 else t).strip().lower()


def run_thinking(clm, out, max_tokens: int = 512, temperature: float = 0.0, enable_thinking: bool = False, cases=None, echo=None) -> dict:
    from deliverance_b200.params import GeneratorParameters

    passed = warnings = 0
    cases = CASES if cases is None else cases
    for case in cases:
        messages, total_ms, total_tokens, r = [], 0.0, 0, None
        for user in case.prompts:
            messages.append(("user", user))
            pb = clm.prompt_builder().with_kwargs({"enable_thinking": bool(enable_thinking)})
            for role, content in messages:
                pb = pb.add_user(content) if role == "user" else pb.add_assistant(content)
            t0 = time.perf_counter()
            r = clm.generate(pb.build(), GeneratorParameters(max_tokens=max_tokens, temperature=temperature))
            total_ms += (time.perf_counter() - t0) * 1e3
            total_tokens += r.generated_tokens
            messages.append(("assistant", r.text))
        ok = case.check(final_answer(r.text_with_special_tokens or r.text))
        passed += ok
        warnings += r.finish_reason.wire == "length"
        row = {"timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat(), "case_id": case.id, "pass": bool(ok),
               "finish_reason": r.finish_reason.name, "generated_tokens": total_tokens, "time_ms": round(total_ms, 3),
               "time_to_first_token_ms": round(r.ttft_ms, 3), "response": r.text_with_special_tokens or r.text}
        out.write(json.dumps(row) + "\n")
        out.flush()
        if echo:
            echo(f"case {case.id}: pass={ok} finish={r.finish_reason.name} generated={total_tokens} time_ms={total_ms:.0f} ttft_ms={r.ttft_ms:.1f}")
    summary = {"passed": passed, "cases": len(cases), "max_token_warnings": warnings}
    if echo:
        echo(f"summary passed={passed}/{len(cases)} max_token_warnings={warnings}")
    return summary


LORA_COLUMNS = ["timestamp", "variant", "model", "case_id", "category", "prompt_chars", "prompt_tokens", "generated_tokens", "total_ms",
                "generation_ms", "tokens_per_second", "response_chars", "finish_reason"]
LORA_PROMPTS = [("explain-1", "writing", "Explain what a hash map is in two sentences."),
                ("code-1", "coding", "Write a Python one-liner that reverses a string."),
                ("math-1", "math", "What is 12 squared minus 44?")]


def run_lora(model_dir: str, adapter_dir: str, out, mode: str = "merge", max_tokens: int = 64, device: str = "auto", prompts=None,
             jsonl=None) -> list:
    """Rows for the base variant, then for the adapted variant. ``merge``: two loads (the second through the merging loader);
    ``hotswap``: one load, the adapter is activated at run time."""
    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.params import GeneratorParameters

    prompts = LORA_PROMPTS if prompts is None else prompts
    w = csv.writer(out)
    w.writerow(LORA_COLUMNS)
    rows = []

    def run_variant(clm, variant):
        for case_id, category, text in prompts:
            ctx = clm.prompt_builder().add_user(text).build()
            t0 = time.perf_counter()
            r = clm.generate(ctx, GeneratorParameters(max_tokens=max_tokens, temperature=0.0))
            total = (time.perf_counter() - t0) * 1e3
            gen_ms = max(total - r.ttft_ms, 1e-9)
            n = r.generated_tokens
            row = [datetime.datetime.now(datetime.timezone.utc).isoformat(), variant, clm.name, case_id, category, len(ctx.prompt), r.prompt_tokens, n,
                   f"{total:.2f}", f"{gen_ms:.2f}", f"{((n - 1) / (gen_ms / 1e3) if n > 1 else 0.0):.2f}", len(r.text or ""), r.finish_reason.wire]
            w.writerow(row)
            out.flush()
            rows.append(dict(zip(LORA_COLUMNS, row), response_text=r.text, token_ids=list(r.token_ids)))
            if jsonl is not None:
                jsonl.write(json.dumps(rows[-1]) + "\n")
                jsonl.flush()

    base = AutoModelForCausalLM.new_builder(model_dir).with_device(device).build()
    run_variant(base, "base")
    if mode == "hotswap":
        base.activate_lora(base.register_lora(adapter_dir))
        run_variant(base, "lora-adapted")
        base.activate_lora(None)
    else:
        del base
        run_variant(AutoModelForCausalLM.new_builder(model_dir).with_device(device).with_lora_adapter(adapter_dir).build(), "lora-adapted")
    return rows


def main(argv: Optional[list] = None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("thinking")
    t.add_argument("--model", required=True)
    t.add_argument("--out", default="-")
    t.add_argument("--max-tokens", type=int, default=512)
    t.add_argument("--temperature", type=float, default=0.0)
    t.add_argument("--enable-thinking", action="store_true")
    t.add_argument("--device", default="auto")
    lo = sub.add_parser("lora")
    lo.add_argument("--model", required=True)
    lo.add_argument("--adapter", required=True)
    lo.add_argument("--mode", default="merge", choices=["merge", "hotswap"])
    lo.add_argument("--out", default="-")
    lo.add_argument("--jsonl-output")
    lo.add_argument("--max-tokens", type=int, default=64)
    lo.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    out = sys.stdout if a.out == "-" else open(a.out, "w", newline="")
    if a.cmd == "thinking":
        from deliverance_b200.api import AutoModelForCausalLM

        clm = AutoModelForCausalLM.new_builder(a.model).with_device(a.device).build()
        run_thinking(clm, out, a.max_tokens, a.temperature, a.enable_thinking, echo=lambda s: print(s, file=sys.stderr))
    else:
        jl = open(a.jsonl_output, "w") if a.jsonl_output else None
        run_lora(a.model, a.adapter, out, a.mode, a.max_tokens, a.device, jsonl=jl)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
