"""Serving benchmark through the HTTP path: N concurrent ``/chat/completions`` streams with a shared prompt prefix.

Default load = the Gemma2-9B-shaped serving configuration: bf16 weights (random init), 128 concurrent streams whose prompts
share a random 1536-token prefix (prefix cache) plus 256 unique tokens each, half of the streams guided by a flat JSON schema
of 8 string / integer fields, the other half sampled with top-p 0.9, 256 generated tokens per stream. The model is served by
the framework's own FastAPI application (uvicorn in a thread, engine runner thread, continuous batching); the load generator
is a separate process (asyncio + aiohttp) so that it does not share the interpreter lock with the server.

Under ``torchrun`` rank 0 serves HTTP and drives the other ranks in lockstep (server/lockstep.py).

    python -m deliverance_b200.bench.serve_bench [--shape gemma2-9b] [--streams 128] [--layers N]

Prints one JSON line: aggregate generated tokens/s, p50 / p95 time to first token, prefix-cache hit counts, engine metrics.
The tokenizer is the byte-level fallback (synthetic models have no vocabulary files): a "token" of the prompt is one byte.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import socket
import subprocess
import sys
import tempfile
import threading
import time


def _schema(rng: random.Random) -> dict:
    props = {}
    for i in range(8):
        # bounded value sets: a random-init model would otherwise emit digits until max_tokens and never close the object
        props[f"f{i}_{rng.randrange(1000)}"] = {"type": "string", "maxLength": 6} if rng.random() < 0.5 else {"enum": [rng.randrange(100) for _ in range(3)]}
    return {"type": "object", "properties": props, "required": list(props), "additionalProperties": False}


def client_main(a) -> int:
    import asyncio

    import aiohttp

    rng = random.Random(a.seed)
    alphabet = "abcdefghijklmnopqrstuvwxyz ,.;"
    prefix = "".join(rng.choice(alphabet) for _ in range(a.prefix))
    schema = _schema(rng)
    bodies = []
    for i in range(a.streams):
        unique = "".join(rng.choice(alphabet) for _ in range(a.unique))
        body = {"messages": [{"role": "user", "content": prefix + unique}], "max_tokens": a.gen, "stream": True, "seed": i}
        if i < int(a.streams * a.guided_frac):
            body["guided_json"] = schema
            body["temperature"] = 0.7
        else:
            body["temperature"] = 0.8
            body["top_p"] = 0.9
        bodies.append(body)
    stats = []

    async def one(session, body):
        t0 = time.perf_counter()
        first = None
        chunks = 0
        text = []
        async with session.post(a.url + "/chat/completions", json=body) as r:
            async for raw in r.content:
                line = raw.decode("utf-8", "replace").strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ch = json.loads(line[6:])
                if "error" in ch:
                    stats.append({"error": ch["error"].get("message", "?")})
                    return
                d = ch["choices"][0].get("delta", {})
                if d.get("content"):
                    if first is None:
                        first = time.perf_counter() - t0
                    chunks += 1
                    text.append(d["content"])
                usage = ch.get("usage")
        stats.append({"ttft": first, "total": time.perf_counter() - t0, "chunks": chunks, "guided": "guided_json" in body, "text": "".join(text)})

    async def run():
        conn = aiohttp.TCPConnector(limit=0)
        async with aiohttp.ClientSession(connector=conn, timeout=aiohttp.ClientTimeout(total=a.timeout)) as s:
            t0 = time.perf_counter()
            await asyncio.gather(*[one(s, b) for b in bodies])
            return time.perf_counter() - t0

    wall = asyncio.run(run())
    ok = [s for s in stats if "error" not in s and s["ttft"] is not None]
    ttft = sorted(s["ttft"] for s in ok)
    valid_json = 0
    for s in ok:
        if s["guided"]:
            try:
                json.loads(s["text"])
                valid_json += 1
            except ValueError:
                pass
    # "completed" = streams that ended without an error; "streams_with_text" = those that delivered at least one non-empty content
    # delta (a random-weight model mostly samples ids that the byte-level fallback tokenizer decodes to nothing, so the
    # unguided half of the load often streams no text at all; the guided half always does)
    out = {"streams": a.streams, "completed": sum(1 for s in stats if "error" not in s), "streams_with_text": len(ok), "errors": [s["error"] for s in stats if "error" in s][:3], "wall_s": wall,
           "ttft_p50_ms": ttft[len(ttft) // 2] * 1e3 if ttft else None, "ttft_p95_ms": ttft[int(len(ttft) * 0.95)] * 1e3 if ttft else None,
           "guided_streams": sum(1 for s in ok if s["guided"]), "guided_parse_as_json": valid_json}
    print("CLIENT " + json.dumps(out), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="gemma2-9b")
    ap.add_argument("--quant", default="bf16", choices=["bf16", "jq4"])
    ap.add_argument("--streams", type=int, default=128)
    ap.add_argument("--prefix", type=int, default=1536)
    ap.add_argument("--unique", type=int, default=256)
    ap.add_argument("--gen", type=int, default=256)
    ap.add_argument("--guided-frac", type=float, default=0.5)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (smaller smoke runs)")
    ap.add_argument("--seed", type=int, default=7)
    ap.add_argument("--timeout", type=float, default=1200.0)
    ap.add_argument("--client", action="store_true")
    ap.add_argument("--url", default="")
    a = ap.parse_args()
    if a.client:
        return client_main(a)

    import torch

    from deliverance_b200.api import CausalLanguageModel
    from deliverance_b200.ckpt.synthetic import SHAPES, SyntheticLoader
    from deliverance_b200.config import parse_config
    from deliverance_b200.engine.engine import Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.parallel.context import TensorParallelContext, TorchCollectives
    from deliverance_b200.tokenizer.auto import AutoTokenizer

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp, control = TensorParallelContext(), None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
        tp = TensorParallelContext(rank, world, TorchCollectives())
        control = TorchCollectives(dist.new_group(backend="gloo"))
        try:
            from deliverance_b200.parallel.fused import FusedTensorParallel

            tp.fused = FusedTensorParallel.create(tp, dev)
        except Exception as e:  # noqa: BLE001
            print(f"[serve_bench] fused TP unavailable: {e}", file=sys.stderr)
    shape = dict(SHAPES[a.shape])
    if a.layers:
        shape["num_hidden_layers"] = a.layers
    cfg = parse_config(dict(shape))
    model = DecoderModel(cfg, dev, torch.bfloat16, tp).load(SyntheticLoader(shape, 0, a.quant == "jq4", dev, dtype=torch.bfloat16))
    per_seq = (a.prefix + a.unique + a.gen + 256 + 31) // 32
    ec = EngineConfig(max_batch_tokens=8192, max_seqs=a.streams, num_pages=a.streams * per_seq + 64)
    ec.kv.max_prefix_tokens = max(4096, a.prefix + a.unique)  # the reference's default caches at most 512 prompt tokens
    ec.kv.policy = "FIXED_BLOCKS"
    eng = Engine(model, ec, eos_ids=(-1,))
    d = tempfile.mkdtemp(prefix="dlv_serve_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(shape, f)
    clm = CausalLanguageModel(model, eng, AutoTokenizer.from_pretrained(d), a.shape)
    clm.eos_ids = set()
    eng.eos_ids = frozenset((-1,))
    if world > 1 and rank != 0:
        from deliverance_b200.server.lockstep import follower_loop

        follower_loop(clm, control)
        return 0

    import uvicorn

    from deliverance_b200.server.app import ModelRegistry, create_app
    from deliverance_b200.server.runner import EngineRunner

    if world > 1:
        from deliverance_b200.server.lockstep import LockstepRunner

        runner = LockstepRunner(clm, control)
    else:
        runner = EngineRunner(clm)
    reg = ModelRegistry()
    reg.generation[clm.name] = runner
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    server = uvicorn.Server(uvicorn.Config(create_app(reg), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    while not server.started:
        time.sleep(0.05)
    cmd = [sys.executable, "-m", "deliverance_b200.bench.serve_bench", "--client", "--url", f"http://127.0.0.1:{port}", "--streams", str(a.streams),
           "--prefix", str(a.prefix), "--unique", str(a.unique), "--gen", str(a.gen), "--guided-frac", str(a.guided_frac), "--seed", str(a.seed),
           "--timeout", str(a.timeout)]
    t0 = time.perf_counter()
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=a.timeout + 60)
    wall = time.perf_counter() - t0
    line = [l for l in p.stdout.splitlines() if l.startswith("CLIENT ")]
    client = json.loads(line[0][7:]) if line else {"error": p.stderr[-2000:]}
    server.should_exit = True
    runner.close()
    m = eng.metrics
    gen_tokens = m["decode_tokens"] + client.get("completed", 0)
    out = {"metric": "serving_generated_tokens_per_s", "value": gen_tokens / client["wall_s"] if client.get("wall_s") else None, "unit": "tokens/s",
           "n_gpus": world, "config": {"model": f"{a.shape}-shape {a.quant}", "streams": a.streams, "shared_prefix_tokens": a.prefix,
                                       "unique_tokens": a.unique, "generated_per_stream": a.gen, "guided_json_fraction": a.guided_frac,
                                       "layers": cfg.num_layers, "path": "HTTP /chat/completions (SSE), byte-level tokenizer"},
           "client": client, "prefix_cache": dict(eng.kv.prefix.metrics),
           "engine": {k: m[k] for k in ("steps", "prefill_steps", "decode_steps", "prefill_tokens", "decode_tokens", "graph_replays")},
           "runner": runner.stats, "wall_with_startup_s": wall}
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
