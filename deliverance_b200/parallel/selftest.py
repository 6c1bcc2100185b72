"""Multi-GPU self-test of the tensor-parallel paths; run one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 \
        -m deliverance_b200.parallel.selftest [--bench]

Checks (1) the fused GEMM + all-reduce epilogue against an fp32 reference built from all-gathered shards, over decode
batch sizes, JQ4 and dense weights, repeated launches and a captured CUDA graph; (2) greedy tokens of a tensor-parallel
Qwen3-shaped model against the same model on one GPU; with ``--bench`` it also times fused vs GEMM + NCCL all-reduce
(device time, max over ranks) and prints the fraction of the NVLink roofline. Rank 0 prints one JSON line per check.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bench", action="store_true")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from deliverance_b200 import ops
    from deliverance_b200.ckpt.jq4 import q4_dequantize, q4_quantize
    from deliverance_b200.ckpt.safetensors_io import Q4Tensor
    from deliverance_b200.ops import LinearWeight
    from deliverance_b200.parallel.context import TensorParallelContext, TorchCollectives
    from deliverance_b200.parallel.fused import FusedTensorParallel

    tp = TensorParallelContext(rank, world, TorchCollectives())
    fused = FusedTensorParallel.create(tp, dev)
    ok_all = True

    def report(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    # ---------------------------------------------------------------- (1) fused linear + all-reduce numerics
    for (N, Kfull, q4) in [(2560, 4096, True), (2560, 9728 // 2 * 2 if world != 8 else 9728, True), (1024, 2048, False)]:
        Kfull = (Kfull // (32 * world)) * 32 * world
        Ks = Kfull // world
        g = torch.Generator().manual_seed(100 + N + Kfull)
        wfull = torch.randn(N, Kfull, generator=g) * 0.05
        wsh = wfull[:, rank * Ks : (rank + 1) * Ks].contiguous()
        if q4:
            p, s = q4_quantize(wsh)
            lw = LinearWeight(Q4Tensor(p, s, (N, Ks))).to(dev)
            wref = q4_dequantize(p, s)
        else:
            lw = LinearWeight(wsh.to(torch.bfloat16)).to(dev, torch.bfloat16)
            wref = wsh.to(torch.bfloat16).float()
        for M in (1, 8, 64, 100):
            xfull = (torch.randn(M, Kfull, generator=g) * 0.5).to(torch.bfloat16)
            x = xfull[:, rank * Ks : (rank + 1) * Ks].contiguous().to(dev)
            part = (x.float().cpu() @ wref.t()).to(dev)
            dist.all_reduce(part)
            ys = [fused.linear_all_reduce(x, lw, "t") for _ in range(3)]
            torch.cuda.synchronize()
            ops.check_status(local)
            err = max(((y.float() - part).norm() / part.norm()).item() for y in ys)
            same = all(torch.equal(ys[0], y) for y in ys[1:])
            gathered = [torch.empty_like(ys[0]) for _ in range(world)]
            dist.all_gather(gathered, ys[0])
            identical = all(torch.equal(gathered[0], t) for t in gathered)
            good = err < 2e-2 and same and identical
            ok_all &= good
            report(check="fused_linear_all_reduce", N=N, K=Kfull, M=M, q4=q4, rel_err=err, repeatable=same, ranks_identical=identical, ok=good)
            # split form: publish-only GEMM, then one row-wise kernel = wait + sum over ranks + residual add + RMSNorm
            if M <= 64 and fused.reduce_mode != "epilogue":
                res0 = (torch.randn(M, N, generator=g) * 0.5).to(torch.bfloat16).to(dev)
                nw = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).to(dev)
                r_ref = res0.clone()
                x_ref = ops.add_rmsnorm(ys[0], r_ref, nw, 1e-6, 0.0, 1.0)
                outs = []
                for _ in range(3):
                    r = res0.clone()
                    xn = fused.linear_reduce_norm(x, lw, r, nw, None, 1e-6, 0.0, 1.0)
                    outs.append((xn, r))
                torch.cuda.synchronize()
                ops.check_status(local)
                good = all(o[0] is not None for o in outs)
                if good:
                    e1 = ((outs[0][0].float() - x_ref.float()).norm() / x_ref.float().norm()).item()
                    e2 = ((outs[0][1].float() - r_ref.float()).norm() / r_ref.float().norm()).item()
                    same = all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs[1:])
                    gathered = [torch.empty_like(outs[0][0]) for _ in range(world)]
                    dist.all_gather(gathered, outs[0][0])
                    identical = all(torch.equal(gathered[0], t) for t in gathered)
                    good = e1 < 1e-2 and e2 < 1e-2 and same and identical
                    report(check="linear_reduce_norm", mode=fused.reduce_mode, N=N, K=Kfull, M=M, q4=q4, rel_err_x=e1, rel_err_residual=e2,
                           repeatable=same, ranks_identical=identical, ok=good)
                else:
                    report(check="linear_reduce_norm", mode=fused.reduce_mode, N=N, K=Kfull, M=M, q4=q4, ok=False, reason="outside the fused path")
                ok_all &= good
    # CUDA graph capture of two fused calls back to back (parity flips between them)
    x = (torch.randn(16, lw.K, device=dev) * 0.5).to(torch.bfloat16)
    ref = fused.linear_all_reduce(x, lw, "g").clone()
    gr = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fused.linear_all_reduce(x, lw, "g")
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.graph(gr):
        y1 = fused.linear_all_reduce(x, lw, "g")
        y2 = fused.linear_all_reduce(x, lw, "g")
    for _ in range(5):
        gr.replay()
    torch.cuda.synchronize()
    ops.check_status(local)
    good = torch.equal(y1, ref) and torch.equal(y2, ref)
    ok_all &= good
    report(check="fused_in_cuda_graph", ok=good, fused_calls=fused.stats["fused"], fallback_calls=fused.stats["fallback"])

    # prefill-size batches: GEMM -> reduce-scatter -> all-gather (only when DLV_TP_SCATTER=1 built the state)
    if fused.scatter is not None:
        for M in (256 * world, 256 * world + 9, 2048 + 256 * world):
            g = torch.Generator().manual_seed(7 + M)
            xs = (torch.randn(M, lw.K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
            part = (xs.float().cpu() @ wref.t()).to(dev)
            dist.all_reduce(part)
            before = fused.stats["scatter"]
            ys = [fused.linear_all_reduce(xs, lw, "s") for _ in range(3)]
            torch.cuda.synchronize()
            ops.check_status(local)
            err = max(((y.float() - part).norm() / part.norm()).item() for y in ys)
            gathered = [torch.empty_like(ys[0]) for _ in range(world)]
            dist.all_gather(gathered, ys[0])
            good = err < 2e-2 and all(torch.equal(ys[0], y) for y in ys[1:]) and all(torch.equal(gathered[0], t) for t in gathered) \
                and fused.stats["scatter"] == before + 3
            ok_all &= good
            report(check="gemm_reduce_scatter_gather", M=M, N=lw.N, K_per_rank=lw.K, rel_err=err, ok=good)
        # sequence-parallel chain: reduce-scatter (own rows only) -> all-gather -> GEMM, repeated without barriers in between
        M = 256 * world + 40
        g = torch.Generator().manual_seed(3)
        xs = (torch.randn(M, lw.K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        part = (xs.float().cpu() @ wref.t()).to(dev)
        dist.all_reduce(part)
        first, count = fused.own_rows(M)
        w_back = LinearWeight((torch.randn(lw.K, lw.N, generator=g) * 0.05).to(torch.bfloat16)).to(dev, torch.bfloat16)
        good = True
        dist.barrier()
        for it in range(3):
            own = fused.linear_reduce_scatter(xs, lw, "sp")
            y = fused.all_gather_linear(own, M, w_back, ordered=True)
            torch.cuda.synchronize()
            ops.check_status(local)
            want = ops.linear(part.to(torch.bfloat16), w_back)
            e1 = ((own.float() - part[first:first + count]).norm() / part.norm()).item()
            e2 = ((y.float() - want.float()).norm() / want.float().norm()).item()
            good = good and own.shape[0] == count and e1 < 2e-2 and e2 < 3e-2
        ok_all &= good
        report(check="reduce_scatter_then_all_gather_gemm", M=M, rel_err_rows=e1, rel_err_chain=e2, ok=good)
        # all-gather -> GEMM: every rank holds its rows of the activations, the weight (same on every rank here) multiplies all rows
        for M in (256 * world, 256 * world + 9):
            g = torch.Generator().manual_seed(11 + M)
            xfull = (torch.randn(M, lw.K, generator=g) * 0.5).to(torch.bfloat16)
            first, count = fused.own_rows(M)
            x_own = xfull[first:first + count].contiguous().to(dev)
            want = (xfull.float() @ wref.t()).to(dev)
            ys = [fused.all_gather_linear(x_own, M, lw) for _ in range(3)]
            torch.cuda.synchronize()
            ops.check_status(local)
            err = max(((y.float() - want).norm() / want.norm()).item() for y in ys)
            good = err < 2e-2 and fused.stats.get("gathered", 0) >= 3
            ok_all &= good
            report(check="all_gather_gemm", M=M, N=lw.N, K=lw.K, rel_err=err, ok=good)

    # ---------------------------------------------------------------- (2) tensor-parallel model vs single GPU
    from deliverance_b200.ckpt.synthetic import SyntheticLoader
    from deliverance_b200.config import parse_config
    from deliverance_b200.engine.engine import Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.params import GeneratorParameters

    shape = dict(model_type="qwen3", vocab_size=4096, hidden_size=1024, intermediate_size=2048 * 2, num_hidden_layers=3,
                 num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=1024, rms_norm_eps=1e-6,
                 rope_theta=1e6, tie_word_embeddings=True)
    cfg = parse_config(dict(shape))
    prompts = [torch.randint(0, 4096, (n,), generator=torch.Generator().manual_seed(5 + n)).tolist() for n in (70, 33, 129)]
    results = {}
    for name, ctx in (("single", TensorParallelContext()), ("tp_nccl", TensorParallelContext(rank, world, TorchCollectives())), ("tp_fused", tp)):
        if name == "tp_fused":
            ctx.fused = fused
        model = DecoderModel(cfg, dev, torch.bfloat16, ctx).load(SyntheticLoader(shape, 3, True, dev, std=0.05), head_quant="Q4")
        ec = EngineConfig(num_pages=256, cuda_graphs=True)
        ec.kv.enabled = False
        eng = Engine(model, ec, eos_ids=(-1,))
        rs = eng.generate_batch(prompts, GeneratorParameters(max_tokens=12))
        results[name] = [r.token_ids for r in rs]
        torch.cuda.synchronize()
        ops.check_status(local)
        dist.barrier()
    agree_nccl = sum(a == b for a, b in zip(results["single"], results["tp_nccl"]))
    agree_fused = sum(a == b for a, b in zip(results["single"], results["tp_fused"]))
    first_tok = all(a[0] == b[0] for a, b in zip(results["single"], results["tp_fused"]))
    # bf16 partial sums are rounded per rank, so long greedy continuations may diverge; the first tokens must agree
    good = first_tok
    ok_all &= good
    report(check="tp_model_tokens", sequences=len(prompts), equal_nccl=agree_nccl, equal_fused=agree_fused, first_token_equal=first_tok, ok=good,
           fused_calls=fused.stats["fused"], fallback_calls=fused.stats["fallback"])

    # sequence-parallel prefill (DLV_TP_SEQ_PARALLEL=1): a prompt long enough for the row-sharded path against the same model on one GPU
    n_long = 256 * world + 17
    if os.environ.get("DLV_TP_SEQ_PARALLEL") == "1" and n_long + 8 <= shape["max_position_embeddings"]:
        long_prompt = [torch.randint(0, 4096, (n_long,), generator=torch.Generator().manual_seed(99)).tolist()]
        toks = {}
        for name, ctx in (("single", TensorParallelContext()), ("tp_sp", tp)):
            model = DecoderModel(cfg, dev, torch.bfloat16, ctx).load(SyntheticLoader(shape, 3, True, dev, std=0.05), head_quant="Q4")
            # a sequence-parallel forward keeps projection and rotary embedding as two kernels; the reference run does the same, so that
            # the comparison of greedy tokens of a random-weight model (near-ties between logits) is between equal roundings
            model.fused_rope = False
            used = []
            plan = model._sp_plan
            model._sp_plan = lambda b, plan=plan, used=used: (used.append(plan(b)), used[-1])[1]
            ec = EngineConfig(num_pages=256, cuda_graphs=False)
            ec.kv.enabled = False
            rs = Engine(model, ec, eos_ids=(-1,)).generate_batch(long_prompt, GeneratorParameters(max_tokens=4))
            toks[name] = (rs[0].token_ids, sum(1 for u in used if u is not None))
            torch.cuda.synchronize()
            ops.check_status(local)
            dist.barrier()
        good = toks["single"][0][0] == toks["tp_sp"][0][0] and toks["tp_sp"][1] >= 1
        ok_all &= good
        report(check="sequence_parallel_prefill_tokens", prompt=n_long, first_token_equal=good, sp_forwards=toks["tp_sp"][1],
               equal_tokens=toks["single"][0] == toks["tp_sp"][0], ok=good)

    # ---------------------------------------------------------------- (2b) one-shot all-reduce and fused MoE combine
    e = ops.require_ext()
    g = torch.Generator().manual_seed(77)
    for rows, Hd in ((1, 2048), (64, 4096), (128, 2560)):
        full = (torch.randn(world, rows, Hd, generator=g) * 0.5).to(torch.bfloat16)
        mine = full[rank].contiguous().to(dev)
        want = full.float().sum(0).to(dev)
        outs = [fused.all_reduce(mine, "ar") for _ in range(3)]
        torch.cuda.synchronize()
        ops.check_status(local)
        err = max(((o.float() - want).norm() / want.norm()).item() for o in outs)
        good = err < 1e-2 and all(torch.equal(outs[0], o) for o in outs[1:])
        ok_all &= good
        report(check="oneshot_all_reduce", rows=rows, H=Hd, rel_err=err, ok=good)
    for (T, E, k, Hd) in ((64, 8, 2, 4096), (32, 128, 8, 2048), (5, 8 * world, 2, 1024)):
        if E % world:
            continue
        ne, e0 = E // world, rank * (E // world)
        logits = torch.randn(T, E, generator=g)
        w_, idx, counts, offsets, perm, pos = e.moe_route(logits.to(dev), k, 0, True)
        ys_full = (torch.randn(T * k, Hd, generator=g) * 0.5).to(torch.bfloat16)  # every rank draws the same rows ...
        ys = ys_full.to(dev)
        lo, hi = int(offsets[e0].item()), int(offsets[e0 + ne].item())
        junk = torch.full_like(ys, float("nan"))
        junk[lo:hi] = ys[lo:hi]  # ... but only holds those of its own experts
        got = fused.moe_combine_all_reduce(junk, pos, w_, T, k, offsets, e0, ne)
        torch.cuda.synchronize()
        ops.check_status(local)
        want = (ys_full.float()[pos.cpu().long()].reshape(T, k, Hd) * w_.cpu().unsqueeze(-1)).sum(1).to(dev)
        err = ((got.float() - want).norm() / want.norm()).item() if got is not None else float("nan")
        good = got is not None and err < 2e-2
        ok_all &= good
        report(check="moe_combine_all_reduce", T=T, E=E, k=k, H=Hd, rel_err=err, ok=good)

    # ---------------------------------------------------------------- (2c) expert-parallel MoE model vs single GPU
    mshape = dict(model_type="qwen3_moe", vocab_size=4096, hidden_size=1024, intermediate_size=2048, num_hidden_layers=2,
                  num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=1024, rms_norm_eps=1e-6,
                  rope_theta=1e6, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True,
                  decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False)
    mcfg = parse_config(dict(mshape))
    mres = {}
    for name, ctx in (("single", TensorParallelContext()), ("ep_fused", tp)):
        model = DecoderModel(mcfg, dev, torch.bfloat16, ctx).load(SyntheticLoader(mshape, 5, True, dev, std=0.05))
        ec = EngineConfig(num_pages=256, cuda_graphs=True)
        ec.kv.enabled = False
        eng = Engine(model, ec, eos_ids=(-1,))
        rs = eng.generate_batch(prompts, GeneratorParameters(max_tokens=8))
        mres[name] = [r.token_ids for r in rs]
        local_experts = [lw.n_local_experts for lw in model.layers if lw.router is not None]
        torch.cuda.synchronize()
        ops.check_status(local)
        dist.barrier()
    first_tok = all(a[0] == b[0] for a, b in zip(mres["single"], mres["ep_fused"]))
    equal = sum(a == b for a, b in zip(mres["single"], mres["ep_fused"]))
    ok_all &= first_tok
    report(check="ep_moe_model_tokens", local_experts=local_experts[0], equal=equal, first_token_equal=first_tok, ok=first_tok,
           fused_calls=fused.stats["fused"], fallback_calls=fused.stats["fallback"])

    # sequence-parallel prefill of the expert-parallel model: attention through reduce-scatter / all-gather, experts through the all-to-all
    n_long = 256 * world + 11
    if os.environ.get("DLV_TP_SEQ_PARALLEL") == "1" and fused.scatter is not None and n_long + 8 <= mshape["max_position_embeddings"]:
        long_prompt = [torch.randint(0, 4096, (n_long,), generator=torch.Generator().manual_seed(98)).tolist()]
        toks = {}
        for name, ctx in (("single", TensorParallelContext()), ("ep_sp", tp)):
            m2 = DecoderModel(mcfg, dev, torch.bfloat16, ctx).load(SyntheticLoader(mshape, 5, True, dev, std=0.05))
            m2.fused_rope = False  # as above: equal roundings on both sides
            used = []
            plan = m2._sp_plan
            m2._sp_plan = lambda b, plan=plan, used=used: (used.append(plan(b)), used[-1])[1]
            ec = EngineConfig(num_pages=256, cuda_graphs=False)
            ec.kv.enabled = False
            rs = Engine(m2, ec, eos_ids=(-1,)).generate_batch(long_prompt, GeneratorParameters(max_tokens=4))
            toks[name] = (rs[0].token_ids, sum(1 for u in used if u is not None))
            torch.cuda.synchronize()
            ops.check_status(local)
            dist.barrier()
        good = toks["single"][0][0] == toks["ep_sp"][0][0] and toks["ep_sp"][1] >= 1
        ok_all &= good
        report(check="sequence_parallel_moe_all_to_all_tokens", prompt=n_long, first_token_equal=toks["single"][0][0] == toks["ep_sp"][0][0],
               sp_forwards=toks["ep_sp"][1], equal_tokens=toks["single"][0] == toks["ep_sp"][0], ok=good)

    # ---------------------------------------------------------------- (2d) expert-parallel all-to-all: token rows sharded over the ranks
    # The model above (expert-parallel weights on this rank) runs one mixture-of-experts layer two ways on the same rows: replicated
    # tokens with local selection + sum over ranks, and own rows only with dispatch / return over peer memory. Router logits are
    # biased from uniform to a Zipf(1.1) load over the experts.
    from deliverance_b200.models.moe import moe_forward, moe_forward_sharded
    from deliverance_b200.parallel.fused import ExpertAllToAll, row_cut

    lw_moe = next(lw for lw in model.layers if lw.router is not None)
    E_, k_ = mcfg.num_experts, mcfg.experts_per_token
    a2a = ExpertAllToAll(tp, dev, lw_moe.n_local_experts, mcfg.hidden_size, cap=1024 * k_)
    router_w = lw_moe.router
    for (T_all, skew) in ((world * 40 + 3, 0.0), (world * 256, 0.0), (world * 256, 1.1)):
        g3 = torch.Generator().manual_seed(77 + T_all)
        x_all = (torch.randn(T_all, mcfg.hidden_size, generator=g3) * 0.5).to(torch.bfloat16).to(dev)
        if skew > 0:  # push the routing towards a Zipf load: add log(rank^-skew) to the router logits through a bias row trick
            bias = torch.log(torch.arange(1, E_ + 1, dtype=torch.float32) ** (-skew)) * 4.0
            x_all[:, 0] = 0  # keep the activations as they are; the bias enters through the router weight's first column
            saved = router_w
            wd = router_w.dense(torch.bfloat16).clone()
            wd[:, 0] = 0
            lw_moe.router = LinearWeight(wd.cpu()).to(dev, torch.bfloat16)
            lw_moe.router.bias = bias.to(dev)
        rpr, first, count = row_cut(T_all, world, rank)
        want = moe_forward(model, 0, lw_moe, x_all)[first:first + count]
        sent0 = a2a.sent_rows
        got = moe_forward_sharded(model, 0, lw_moe, x_all[first:first + count].contiguous(), a2a, T_all)
        torch.cuda.synchronize()
        ops.check_status(local)
        err = ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-9)).item() if count else 0.0
        good = err < 5e-3
        ok_all &= good
        sent = a2a.sent_rows - sent0
        report(check="ep_all_to_all_dispatch_grouped_gemm_combine", tokens=T_all, own_rows=count, zipf=skew, rel_err=err, ok=good,
               nvlink_bytes_per_rank_a2a=2 * sent * (world - 1) // world * mcfg.hidden_size * 2,
               nvlink_bytes_per_rank_replicated=2 * (world - 1) * T_all * mcfg.hidden_size * 2 // world)
        if skew > 0:
            lw_moe.router = saved
        dist.barrier()

    # ---------------------------------------------------------------- (3) timing
    if a.bench:
        N, Kfull = 2560, 9728 // (32 * world) * 32 * world
        Ks = Kfull // world
        copies = []
        for c in range(24):
            w = torch.randn(N, Ks, device=dev) * 0.02
            p, s = ops.q4_quantize(w)
            copies.append(LinearWeight(Q4Tensor(p, s, (N, Ks))).to(dev))
        for M in (1, 8, 64):
            x = (torch.randn(M, Ks, device=dev) * 0.5).to(torch.bfloat16)
            res = {}
            for mode in ("fused", "gemm+nccl"):
                def run(i):
                    if mode == "fused":
                        return fused.linear_all_reduce(x, copies[i % 24], "b")
                    y = ops.linear(x, copies[i % 24])
                    dist.all_reduce(y)
                    return y
                for i in range(24):
                    run(i)
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(48):
                    run(i)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) * 1e3 / 48], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res[mode] = t.item()
            # roofline: slower of weight bytes at the measured HBM rate and bytes this GPU must send over NVLink at 770 GB/s
            hbm_us = N * Ks * 0.5625 / 6454.3e3
            nvl_us = (world - 1) * M * N * 2 / 770e3
            roof = max(hbm_us, nvl_us)
            # the same projection followed by the residual add + norm of the layer: fused epilogue + norm kernel, split form, GEMM + NCCL + norm
            resb = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
            nwb = torch.ones(N, dtype=torch.bfloat16, device=dev)
            res2 = {}
            for mode in ("epilogue+norm", "split", "gemm+nccl+norm"):
                if mode == "split" and fused.reduce_mode == "epilogue":
                    continue

                def run2(i):
                    if mode == "split":
                        return fused.linear_reduce_norm(x, copies[i % 24], resb, nwb, None, 1e-6, 0.0, 0.0)
                    if mode == "epilogue+norm":
                        y = fused.linear_all_reduce(x, copies[i % 24], "b")
                    else:
                        y = ops.linear(x, copies[i % 24])
                        dist.all_reduce(y)
                    return ops.add_rmsnorm(y, resb, nwb, 1e-6, 0.0, 0.0)
                for i in range(24):
                    run2(i)
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(48):
                    run2(i)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) * 1e3 / 48], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res2[mode] = t.item()
            report(check="bench_linear_all_reduce", world=world, M=M, N=N, K_per_rank=Ks, fused_us=res["fused"], gemm_nccl_us=res["gemm+nccl"],
                   roofline_us=roof, fused_frac_of_roofline=roof / res["fused"], speedup_vs_nccl=res["gemm+nccl"] / res["fused"],
                   with_norm_us=res2, reduce_mode=fused.reduce_mode)
        # prefill-size: GEMM -> reduce-scatter -> all-gather against GEMM + NCCL all-reduce (needs DLV_TP_SCATTER=1)
        if fused.scatter is not None:
            Np, Kp = 4096, 14336 // (32 * world) * 32
            wp = [LinearWeight((torch.randn(Np, Kp, device=dev) * 0.02).to(torch.bfloat16)).to(dev, torch.bfloat16) for _ in range(4)]
            for M in (2048, 4096):
                if M < 256 * world:
                    continue
                x = (torch.randn(M, Kp, device=dev) * 0.5).to(torch.bfloat16)
                res = {}
                for mode in ("scatter", "gemm+nccl"):
                    def run(i):
                        if mode == "scatter":
                            return fused.linear_all_reduce(x, wp[i % 4], "p")
                        y = ops.linear(x, wp[i % 4])
                        dist.all_reduce(y)
                        return y
                    for i in range(4):
                        run(i)
                    torch.cuda.synchronize()
                    dist.barrier()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for i in range(16):
                        run(i)
                    e1.record()
                    torch.cuda.synchronize()
                    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / 16], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    res[mode] = t.item()
                ops.check_status(local)
                # roofline: slower of the GEMM at the measured cuBLAS bf16 rate and the bytes a GPU must send (partials to the owners,
                # reduced rows to everyone: 2 (n - 1) / n of the output) at 770 GB/s
                flop_us = 2.0 * M * Np * Kp / 1.59e9
                nvl_us = 2.0 * (world - 1) / world * M * Np * 2 / 770e3
                roof = max(flop_us, nvl_us)
                report(check="bench_gemm_reduce_scatter_gather", world=world, M=M, N=Np, K_per_rank=Kp, scatter_us=res["scatter"],
                       gemm_nccl_us=res["gemm+nccl"], roofline_us=roof, frac_of_roofline=roof / res["scatter"],
                       speedup_vs_nccl=res["gemm+nccl"] / res["scatter"])
        # fused MoE combine + all-reduce against the local combine followed by the NCCL all-reduce
        for (T, E, k, Hd) in ((64, 8 * world if world > 8 else 8 if 8 % world == 0 else world, 2, 4096), (32, 128 if 128 % world == 0 else 16 * world, 8, 2048)):
            ne, e0 = E // world, rank * (E // world)
            g2 = torch.Generator().manual_seed(9)
            w_, idx, counts, offsets, perm, pos = e.moe_route(torch.randn(T, E, generator=g2).to(dev), k, 0, True)
            ys = (torch.randn(T * k, Hd, generator=g2) * 0.5).to(torch.bfloat16).to(dev)
            res = {}
            for mode in ("fused", "combine+nccl"):
                def run():
                    if mode == "fused":
                        return fused.moe_combine_all_reduce(ys, pos, w_, T, k, offsets, e0, ne)
                    y = e.moe_combine(ys, pos, w_, T, k, offsets, e0, ne)
                    dist.all_reduce(y)
                    return y
                for _ in range(10):
                    run()
                torch.cuda.synchronize()
                dist.barrier()
                e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0_.record()
                for _ in range(50):
                    run()
                e1_.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0_.elapsed_time(e1_) * 1e3 / 50], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res[mode] = t.item()
            nvl_us = (world - 1) * T * Hd * 2 / 770e3  # bytes this GPU sends at the measured peer-copy rate
            report(check="bench_moe_combine_all_reduce", world=world, T=T, E=E, k=k, H=Hd, fused_us=res["fused"], combine_nccl_us=res["combine+nccl"],
                   nvlink_roofline_us=nvl_us, speedup_vs_nccl=res["combine+nccl"] / res["fused"])
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok_all else 1


if __name__ == "__main__":
    sys.exit(main())
