"""Tokenizer throughput and identity check.

    python -m deliverance_b200.tokenizer.benchmark --model-dir DIR [--text-file FILE] [--repeat 64] [--iterations 200]

Encodes a text ``iterations`` times and prints tokens, characters, a SHA-256 over the token ids (4 bytes each, big endian,
signed: the same digest the reference's tokenizer comparison prints, grace/scripts/hf_fast_tokenizer_benchmark.py:11-16, so a
run of either side can be compared by hash) and mean time / characters per second / tokens per second. It also decodes the ids
incrementally, token by token, and checks that the pieces concatenate to the one-shot decode (the streaming path of the server).
"""
from __future__ import annotations

import argparse
import hashlib
import time

DEFAULT_TEXT = ("The quick brown fox jumps over the lazy dog. Ünïcödé: 你好，世界! 12345 + 67890 = 80235.\n"
                "def f(x):\n    return {'k': [x, x ** 2]}  # code\n\t<|tag|> </s> émoji 🙂\n")


def ids_sha256(ids) -> str:
    h = hashlib.sha256()
    for t in ids:
        h.update(int(t).to_bytes(4, byteorder="big", signed=True))
    return h.hexdigest()


def run(tokenizer, text: str, warmup: int = 5, iterations: int = 50) -> dict:
    from .auto import IncrementalDetokenizer

    ids = tokenizer.encode(text)
    for _ in range(warmup):
        tokenizer.encode(text)
    t0 = time.perf_counter()
    n = 0
    for _ in range(iterations):
        n += len(tokenizer.encode(text))
    dt = time.perf_counter() - t0
    det = IncrementalDetokenizer(tokenizer, skip_special=False)
    t1 = time.perf_counter()
    pieces = "".join(det.push(t) for t in ids)
    d_dt = time.perf_counter() - t1
    return {"ids_sha256": ids_sha256(ids), "tokens": len(ids), "chars": len(text), "bytes": len(text.encode("utf-8")),
            "mean_ms": dt / max(1, iterations) * 1e3, "chars_s": len(text) * iterations / dt, "tokens_s": n / dt,
            "incremental_decode_tokens_s": len(ids) / max(d_dt, 1e-9), "incremental_equals_decode": pieces == tokenizer.decode(ids)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--text-file")
    ap.add_argument("--repeat", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iterations", type=int, default=200)
    a = ap.parse_args()
    from .auto import AutoTokenizer

    text = (open(a.text_file, encoding="utf-8").read() if a.text_file else DEFAULT_TEXT) * a.repeat
    for k, v in run(AutoTokenizer.from_pretrained(a.model_dir), text, a.warmup, a.iterations).items():
        print(f"{k}={v:.3f}" if isinstance(v, float) else f"{k}={v}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
