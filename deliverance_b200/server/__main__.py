"""``python -m deliverance_b200.server --model DIR [--embedding-model DIR] [--port 8080]`` (multi-model: repeat ``--model``).

Under ``torchrun`` every rank loads its tensor-parallel shard; rank 0 serves HTTP and broadcasts each step's admissions to
the other ranks, which run the same engine in lockstep."""
from __future__ import annotations

import argparse
import os


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", action="append", default=[], help="model directory (repeatable)")
    ap.add_argument("--config", help=".properties (or .json) file in the reference's key layout: models, KV cache, auth, port")
    ap.add_argument("--models-root", default=os.environ.get("DELIVERANCE_HOME", "~/.deliverance"), help="where --config model names are looked up")
    ap.add_argument("--embedding-model", action="append", default=[])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--output-head-quantization", default=None)
    ap.add_argument("--reasoning-field", default="openai", choices=["openai", "vllm"])
    ap.add_argument("--basic-user", default=os.environ.get("DELIVERANCE_BASIC_USER"))
    ap.add_argument("--basic-password", default=os.environ.get("DELIVERANCE_BASIC_PASSWORD"))
    ap.add_argument("--jwt-secret", default=os.environ.get("DELIVERANCE_JWT_SECRET"))
    ap.add_argument("--max-seqs", type=int, default=128)
    ap.add_argument("--max-queue", type=int, default=0, help="refuse new requests with 429 while this many are in flight (0: no limit)")
    ap.add_argument("--decode-interleave", type=int, default=0,
                    help="after this many consecutive prompt-chunk steps run one decode step for the running sequences (0: prompts first)")
    a = ap.parse_args()
    conf = None
    head_quant, lora, kv = {}, {}, None
    if a.config:
        from .config import load_server_config

        conf = load_server_config(a.config)
        kv = conf.kv_settings() if conf.kv else None
        for e in conf.models:
            d = e.resolve_dir(a.models_root)
            if e.inference_type == "GENERATION":
                a.model.append(d)
                head_quant[d], lora[d] = e.output_head_quantization, e.lora_adapter
            else:
                a.embedding_model.append(d)
        a.port = conf.port or a.port
        a.reasoning_field = conf.reasoning_field or a.reasoning_field
        a.basic_user, a.basic_password = conf.basic_user or a.basic_user, conf.basic_password or a.basic_password
        a.jwt_secret = conf.jwt_secret or a.jwt_secret
        if conf.ignored:
            print(f"[server] config keys without an equivalent here: {', '.join(sorted(conf.ignored))}", flush=True)
    if not a.model and not a.embedding_model:
        ap.error("--model or --config with at least one model is required")
    import uvicorn

    from ..api import AutoModelForCausalLM
    from ..embedding import AutoModelForEmbeddings
    from .app import ModelRegistry, ServerSettings, create_app
    from .runner import EngineRunner

    world = int(os.environ.get("WORLD_SIZE", "1"))
    tp = control = placement = None
    if world > 1:  # one process per GPU: NCCL for tensors, a gloo side group for the control commands
        import torch
        import torch.distributed as dist

        from ..parallel.context import TensorParallelContext, TorchCollectives

        if len(a.model) != 1:
            raise SystemExit("tensor-parallel serving hosts exactly one generation model")
        cuda = torch.cuda.is_available() and a.device != "cpu"
        if cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            if os.environ.get("DLV_AFFINITY", "off") != "off":  # opt-in: pin this rank to the cores of its GPU's NUMA node
                from ..utils.affinity import place_local_rank

                placement = place_local_rank(int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("LOCAL_WORLD_SIZE", world)))
        dist.init_process_group("nccl" if cuda else "gloo")
        control = TorchCollectives(dist.new_group(backend="gloo"))
        tp = TensorParallelContext(dist.get_rank(), world, TorchCollectives())
        if cuda and os.environ.get("DLV_FUSED_TP", "1") != "0":
            try:  # tensor-parallel sums inside the GEMM epilogue over NVLink peer memory; NCCL all-reduce otherwise
                from ..parallel.fused import FusedTensorParallel

                tp.fused = FusedTensorParallel.create(tp, torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
            except Exception as e:  # noqa: BLE001
                print(f"[server] fused tensor parallelism unavailable, using NCCL all-reduce: {e}", flush=True)
    reg = ModelRegistry()
    if int(os.environ.get("RANK", "0")) == 0:
        from ..parallel.gossip import observer_from_env

        reg.membership = observer_from_env(f"server-{os.getpid()}")  # None unless the host's gossip agent started this process
    for d in a.model:
        b = AutoModelForCausalLM.new_builder(d).with_device(a.device).with_output_head_quantization(head_quant.get(d) or a.output_head_quantization)
        if kv is not None:
            b.with_kv_cache_settings(kv)
        if lora.get(d):
            b.with_lora_adapter(lora[d])
        b.conf.max_seqs = a.max_seqs
        b.conf.decode_interleave = a.decode_interleave
        if tp is not None:
            b.with_tensor_parallel_context(tp)
        clm = b.build()
        if conf is not None and conf.kv_disk_dir and tp is not None:
            # every rank would have to find the same prefixes on disk (a rank that misses a file would run a different batch)
            print("[server] deliverance.kv.disk-dir is ignored under tensor parallelism", flush=True)
        elif conf is not None and conf.kv_disk_dir:
            clm.engine.kv.attach_disk(os.path.join(os.path.expanduser(conf.kv_disk_dir), clm.name),
                                      "MSE_TURBOQUANT" if conf.kv.get("compression") == "MSE_TURBOQUANT" else "LZ4", conf.kv_turboquant_bits or 4)
        if tp is None:
            reg.generation[clm.name] = EngineRunner(clm)
        elif tp.rank == 0:
            from .lockstep import LockstepRunner

            reg.generation[clm.name] = LockstepRunner(clm, control)
        else:
            from .lockstep import follower_loop

            follower_loop(clm, control)
            return 0
    if tp is not None:
        backend = "nccl + fused peer-memory epilogues" if getattr(tp, "fused", None) is not None else ("nccl" if cuda else "gloo")
        reg.tp_status = lambda: {"enabled": True, "size": world, "rank": 0, "backend": backend, "membership": "static",
                                 "placement": None if placement is None else placement.to_json()}
    for d in a.embedding_model:
        reg.embedding[os.path.basename(os.path.normpath(d))] = AutoModelForEmbeddings.from_pretrained(d, a.device)
    settings = ServerSettings(reasoning_field=a.reasoning_field, basic_user=a.basic_user, basic_password=a.basic_password, jwt_secret=a.jwt_secret,
                              max_queue=a.max_queue)
    try:
        uvicorn.run(create_app(reg, settings), host=a.host, port=a.port, log_level="info")
    finally:
        for r in reg.generation.values():  # also tells tensor-parallel followers to stop
            r.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
