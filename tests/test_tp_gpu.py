"""Tensor parallelism on real GPUs (2 ranks): fused GEMM + all-reduce numerics, CUDA-graph replay, TP model vs single GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_selftest():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", "-m", "deliverance_b200.parallel.selftest"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert lines and all(l["ok"] for l in lines if "ok" in l)
    assert any(l["check"] == "fused_in_cuda_graph" for l in lines)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_gemm_reduce_scatter():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, DLV_TP_SCATTER="1", DLV_TP_SEQ_PARALLEL="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29519", "-m", "deliverance_b200.parallel.selftest"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    scat = [l for l in lines if l.get("check") == "gemm_reduce_scatter_gather"]
    assert len(scat) == 3 and all(l["ok"] for l in scat)
    assert any(l.get("check") == "reduce_scatter_then_all_gather_gemm" and l["ok"] for l in lines)
    assert any(l.get("check") == "sequence_parallel_prefill_tokens" and l["ok"] for l in lines)
    gath = [l for l in lines if l.get("check") == "all_gather_gemm"]
    assert len(gath) == 2 and all(l["ok"] for l in gath)
    a2a = [l for l in lines if l.get("check") == "ep_all_to_all_dispatch_grouped_gemm_combine"]
    assert len(a2a) == 3 and all(l["ok"] for l in a2a) and any(l["zipf"] > 0 for l in a2a)
    assert any(l.get("check") == "sequence_parallel_moe_all_to_all_tokens" and l["ok"] for l in lines)
