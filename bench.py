#!/usr/bin/env python
"""Headline benchmark: Qwen3-4B-shaped dense decoder in JQ4, prefill of 2048 random tokens then decode, on N B200s.

N > 1 (``--parallelism``): ``tp`` (the default) shards one engine over the GPUs with the fused tensor-parallel kernels (strong
scaling: the same batch, lower latency per step); ``dp`` runs one engine replica per GPU with the full batch each (weak scaling,
no communication), an explicit extra.

One "step" is one decode step of the whole batch (default 64 sequences, one new token each) after a real 2048-token
prefill; ``value`` is decode tokens/s of the whole job (batch / step time, device-timed with CUDA events, max over ranks).
``e2e`` is the same steps driven through ``Engine.step()`` — every step copies that step's inputs from pinned host memory
and reads the sampled tokens back. ``extras`` carries prefill tokens/s, TTFT and the batch-1 / batch-8 decode rates of the
same configuration. Weights are random-init N(0, 0.02) quantised to JQ4 on the device; prompts are uniform random ids.

``--impl reference`` times the reference's own native decode kernels (its C SIMD library, unmodified, built with gcc) on the
host CPU over the same projection list; the Java engine around them needs a JDK, Maven and the network and cannot be built.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

_ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, _ROOT)

# published reference number this benchmark is compared with: Qwen3-4B-JQ4 decode, single request, CPU (median of the
# seven prompts in benchmarks/runs/2026-08-11-a17cc22-dirty-run-qwen-single-benchmark-014652/qwen-single-benchmark.csv:2-8)
REFERENCE_DECODE_TOK_S = 12.06


def reference_arm(args) -> int:
    """The reference's own native decode kernels (unmodified C, built with gcc from ``baseline/_ref/native_simd``) on the host CPU:
    see ``deliverance_b200/bench/reference_arm.py``. The Java engine around them cannot be built here (no JDK / Maven / network)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:  # the reference is CPU-only: under torchrun the extra ranks would only compete for the same host cores
        return 0
    from deliverance_b200.bench import reference_arm as ra
    from deliverance_b200.ckpt.synthetic import SHAPES

    try:
        r = ra.run(args, SHAPES[args.shape])
    except Exception as e:  # noqa: BLE001 - no gcc, sources not installed, ...
        print(json.dumps({"impl": "reference", "unavailable": f"reference native kernels could not be built or run: {type(e).__name__}: {e}"[:300],
                          "n_gpus": args.gpus}))
        return 0
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": r["tok_s"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": r["tokens_timed"], "warmup": max(1, min(args.warmup, 3)), "ms_per_step": r["ms_per_token"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": r["tok_s"] / REFERENCE_DECODE_TOK_S, "dtype": "int8-block activations x JQ4 (4-bit) weights, fp32 accumulate",
        "data": "synthetic (random packed JQ4 blocks and scales of the benchmark shape)",
        "reference_class": "native-kernels-only (no attention, no JVM): upper bound of the reference",
        "config": {"model": f"{args.shape}-shape jq4", "global_batch": args.batch, "seq_len": args.prompt_len,
                   "parallelism": "host CPU, %d threads (%s); the reference has no GPU path that runs here and no request batching: "
                                  "concurrent requests are independent single-token forwards sharing the cores" % (r["threads"], r["isa"]),
                   "kernel": "gemm_q8_q4 (native/src/main/c/simd/vector_simd.c:595) over q|k|v, o, gate|up, down of every layer + the JQ4 head, per token"},
        "e2e": {"value": r["tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "host memory only: nothing is copied to or from a GPU"},
        "gpu_launches": 0}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.path = tempfile.mktemp(prefix="dlv_clocks_", suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.fh.close()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power), "samples": len(sm),
                "reasons": sorted(reasons)}


def _shutdown(dist, eng) -> None:
    """Leave cleanly, and leave in any case: settle the step in flight, drop the captured graphs (they hold NCCL work when the
    all-reduce runs through NCCL), then tear the process group down under a timer. A communicator teardown that blocks (seen
    once with NCCL collectives captured in CUDA graphs) must not keep eight GPUs busy after the result line is printed."""
    import threading

    import torch

    threading.Timer(45.0, lambda: os._exit(0)).start() if dist is not None else None
    try:
        if eng is not None:
            eng._drain()
            torch.cuda.synchronize()
            eng._graphs.clear()
        if dist is not None:
            torch.cuda.synchronize()
            dist.barrier()
            dist.destroy_process_group()
    finally:
        if dist is not None:
            sys.stdout.flush()
            os._exit(0)  # also ends the timer thread


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="own", choices=["own", "reference", "torch"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--shape", default="qwen3-4b")
    ap.add_argument("--quant", default="jq4", choices=["jq4", "bf16"])
    ap.add_argument("--no-extras", action="store_true", help="skip the batch-1 / batch-8 decode phases")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--parallelism", default="auto", choices=["auto", "dp", "tp"],
                    help="N > 1: tp (default) = one engine over N GPUs (tensor parallel, --batch sequences in total, strong scaling); "
                         "dp = one engine replica per GPU, --batch sequences each (weak scaling, no communication)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    from deliverance_b200 import ops
    from deliverance_b200.ckpt.synthetic import SHAPES, SyntheticLoader
    from deliverance_b200.config import parse_config
    from deliverance_b200.engine.engine import FINISHED, Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.parallel.context import TensorParallelContext, TorchCollectives
    from deliverance_b200.params import GeneratorParameters

    tp = TensorParallelContext()
    dist = None
    mode = args.parallelism
    if mode == "auto":
        mode = "tp"  # the benchmark configuration is tensor parallel at every N; replicas (dp) are an explicit extra
    replicas = world if (world > 1 and mode == "dp") else 1
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if world > 1 and mode == "tp":
        tp = TensorParallelContext(rank, world, TorchCollectives())
        if args.impl == "own" and args.comm in ("auto", "fused"):
            try:
                from deliverance_b200.parallel.fused import FusedTensorParallel

                tp.fused = FusedTensorParallel.create(tp, dev)
            except Exception as e:  # noqa: BLE001
                if args.comm == "fused":
                    raise
                if rank == 0:
                    print(f"[bench] fused TP path unavailable ({type(e).__name__}: {e}); using NCCL all-reduce", file=sys.stderr)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.impl == "torch":  # library baseline: cuBLAS + SDPA + NCCL, bf16 weights, none of this package's kernels
        from deliverance_b200.bench.torch_baseline import run as torch_run

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        r = torch_run(args, dev, rank, world, SHAPES[args.shape], sync_all, max_over_ranks)
        clocks = sampler.stop() if rank == 0 else {}
        if rank == 0:
            print(json.dumps({"impl": "torch-baseline", "metric": "decode_tokens_per_s", "value": r["decode_tok_s"], "unit": "tokens/s",
                              "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": r["decode_tok_s"] / REFERENCE_DECODE_TOK_S,
                              "dtype": "bf16", "data": "synthetic (uniform random prompts, random-init N(0,0.02) bf16 weights)",
                              "config": {"model": f"{args.shape}-shape bf16", "global_batch": args.batch, "seq_len": args.prompt_len,
                                         "parallelism": f"tp{args.gpus}", "kernels": "cuBLAS + torch SDPA + NCCL, decode step in a CUDA graph"},
                              "clocks": clocks, "extras": {"prefill_tok_s": r["prefill_tok_s"], "prefill_ms": r["prefill_ms"]}}))
        _shutdown(dist, None)
        return 0

    ops.require_ext()
    shape = SHAPES[args.shape]
    cfg = parse_config(dict(shape))
    t0 = time.time()
    loader = SyntheticLoader(shape, seed=0, quantize=args.quant == "jq4", device=dev, dtype=torch.bfloat16)
    model = DecoderModel(cfg, dev, torch.bfloat16, tp).load(loader, head_quant="Q4" if args.quant == "jq4" else None)
    B, P = args.batch, args.prompt_len
    total_steps = args.warmup + 2 * args.steps + 16
    pages_per_seq = (P + 3 * total_steps + 64 + 31) // 32
    econf = EngineConfig(max_batch_tokens=8192, max_seqs=max(B, 1), num_pages=B * pages_per_seq + 8, cuda_graphs=not args.no_graphs)
    econf.kv.enabled = False  # random prompts share nothing; the prefix cache is exercised by the serving benchmark
    eng = Engine(model, econf, eos_ids=(-1,))
    torch.cuda.synchronize()
    build_s = time.time() - t0

    g = torch.Generator().manual_seed(1234 + (rank if replicas > 1 else 0))  # replicas serve different prompts
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    pinned = prompts.to(torch.int32).pin_memory()

    # ---------------------------------------------------------------- prefill (device-timed, includes first-token sampling)
    params = GeneratorParameters(temperature=0.0)
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    reqs = [eng.add_request(pinned[i].tolist(), GeneratorParameters(temperature=0.0)) for i in range(B)]
    while any(len(r.output) == 0 for r in reqs):
        eng.step()
    ev1.record()
    sync_all()
    prefill_ms = max_over_ranks(ev0.elapsed_time(ev1))
    ttfts = sorted((r.t_first - r.t_submit) * 1e3 for r in reqs)
    ops.check_status(local_rank)

    # ---------------------------------------------------------------- decode: warm-up (captures the CUDA graph)
    for _ in range(args.warmup):
        eng.step()
    sync_all()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    # (1) end to end through Engine.step(): pinned-host inputs -> H2D, graph replay, argmax, D2H of the sampled tokens
    h2d0 = eng.metrics.get("h2d_bytes", 0)
    l0 = eng.metrics["kernel_launches"] + 0
    sync_all()
    ev0.record()
    for _ in range(args.steps):
        eng.step()
    ev1.record()
    sync_all()
    e2e_ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
    h2d_per_step = (eng.metrics.get("h2d_bytes", 0) - h2d0) // args.steps
    d2h_per_step = B * 8  # int64 token id per sequence

    # (2) device-only: replay the captured decode step + sampling kernel with the inputs already on the device.
    #     Weights (>= 2 GB per rank) exceed the 126 MB L2, so every step streams them from HBM again.
    bucket = next(b for b in sorted(eng._graphs) if b >= B) if eng._graphs else None
    launches_per_step = None
    if bucket is not None:
        gr = eng._graphs[bucket]
        launches_per_step = gr["launches"] + 1
        # The context grows here as it did in (1): step i runs at the positions of the end-to-end loop's step i (the last
        # args.steps positions of every sequence, whose pages exist already), staged on the device before the clock starts.
        gb = gr["batch"]
        ps_ = eng.page_size
        back = torch.arange(args.steps - 1, -1, -1, device=gb.positions.device, dtype=torch.int32).unsqueeze(1)
        pos_all = (gb.positions.unsqueeze(0) - back).clamp_(min=0)                                  # [steps, bucket]
        page_all = torch.gather(gb.block_tables.unsqueeze(0).expand(args.steps, -1, -1), 2, (pos_all // ps_).long().unsqueeze(2)).squeeze(2)
        slots_all = page_all.long() * ps_ + (pos_all % ps_).long()
        ctx_all = torch.where(gb.ctx_len.unsqueeze(0) > 1, pos_all + 1, torch.ones_like(pos_all))  # padded rows keep their context of 1
        sync_all()
        ev0.record()
        for i in range(args.steps):
            gb.positions.copy_(pos_all[i])
            gb.slots.copy_(slots_all[i])
            gb.ctx_len.copy_(ctx_all[i])
            gr["graph"].replay()
            eng._greedy(gr["logits"])
        ev1.record()
        sync_all()
        dev_ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
    else:
        dev_ms = e2e_ms
        launches_per_step = (eng.metrics["kernel_launches"] - l0) // max(1, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    ops.check_status(local_rank)

    extras = {"prefill_tok_s": B * P / (prefill_ms / 1e3), "prefill_ms": prefill_ms, "ttft_ms_p50": ttfts[len(ttfts) // 2],
              "ttft_ms_max": ttfts[-1], "model_build_s": build_s, "weight_bytes_per_rank": model.weight_bytes(),
              "context_at_timing": f"{P + args.warmup + 1}..{P + args.warmup + args.steps} (grows by one token per timed step in both arms)"}

    # ---------------------------------------------------------------- extras: batch 8 and batch 1 decode on the same engine
    if not args.no_extras:
        for nb in (8, 1):
            if nb >= B:
                continue
            for r in reqs[nb:]:
                if r.state != FINISHED:
                    eng.abort(r)
            for _ in range(max(3, args.warmup // 2)):
                eng.step()
            sync_all()
            ev0.record()
            for _ in range(args.steps):
                eng.step()
            ev1.record()
            sync_all()
            ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
            extras[f"decode_tok_s_b{nb}_e2e"] = nb / (ms / 1e3)
            gr = eng._graphs.get(nb)
            if gr is not None:
                sync_all()
                ev0.record()
                for _ in range(args.steps):
                    gr["graph"].replay()
                    eng._greedy(gr["logits"])
                ev1.record()
                sync_all()
                ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
                extras[f"decode_tok_s_b{nb}"] = nb / (ms / 1e3)
        if replicas > 1:
            extras["scope"] = "per replica (one GPU)"
        if "decode_tok_s_b1" in extras:
            extras["vs_baseline_b1"] = extras["decode_tok_s_b1"] / REFERENCE_DECODE_TOK_S

    value = replicas * B / (dev_ms / 1e3)  # replicas: every rank decodes its own B sequences; dev_ms is the slowest rank's step
    if replicas > 1:
        par = f"dp{world}"  # one engine replica per GPU; --parallelism tp shards one engine over the GPUs instead
    elif cfg.num_experts == 0 or args.gpus == 1 or cfg.num_experts % args.gpus:
        par = f"tp{args.gpus}"
    else:
        par = f"tp{args.gpus} attention + ep{args.gpus} experts"
    if rank == 0:
        out = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak" if replicas > 1 else "strong",
            "vs_baseline": value / REFERENCE_DECODE_TOK_S, "dtype": "bf16 activations x JQ4 (4-bit) weights" if args.quant == "jq4" else "bf16",
            "data": "synthetic (uniform random prompts, random-init N(0,0.02) weights quantised to JQ4)",
            "config": {"model": f"{args.shape}-shape {args.quant}", "global_batch": B * replicas, "seq_len": P, "decode_tokens_timed": args.steps,
                       "parallelism": par,
                       "l2": "per-step weight stream (>2 GB/rank) exceeds the 126 MB L2; no flush needed",
                       "comm": ("fused-p2p" if tp.fused is not None else "nccl") if tp.enabled else "none",
                       "baseline_note": "reference number is single-request CPU decode (it has no request batching)"},
            "clocks": clocks,
            "e2e": {"value": replicas * B / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h2d_per_step) * replicas, "d2h_bytes_per_step": int(d2h_per_step) * replicas},
            "gpu_launches": int(launches_per_step * args.steps) * replicas,
            "extras": extras,
        }
        try:  # fraction of the measured roofline (copy bandwidth / cuBLAS rate of this pool) for the timed decode step
            from deliverance_b200.bench.roofline import report

            rf = report(cfg, B, P + args.warmup + args.steps // 2, args.quant, world if tp.enabled else 1, dev_ms)
            out["roofline"] = {k: rf[k] for k in ("target_ms", "bound", "fraction", "hbm_ms", "tensor_ms", "nvlink_ms", "denominators")}
            from deliverance_b200.bench.roofline import prefill_report

            pf = prefill_report(cfg, B, P, args.quant, world if tp.enabled else 1, prefill_ms)
            out["roofline"]["prefill"] = {k: pf[k] for k in ("target_ms", "bound", "fraction")}
        except Exception as e:  # noqa: BLE001 - reporting only
            out["roofline"] = {"error": repr(e)}
        print(json.dumps(out), flush=True)
    _shutdown(dist, eng)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
