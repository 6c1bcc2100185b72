"""GPU model paths against the CPU fp32 oracle: MoE routing kernels, Mamba2 chunked scan, whole models through the engine."""
import pytest
import torch

from deliverance_b200 import ops
from deliverance_b200.ckpt.loader import WeightLoader
from deliverance_b200.ckpt.tiny import write_tiny_model
from deliverance_b200.config import load_config
from deliverance_b200.engine.engine import Engine, EngineConfig
from deliverance_b200.models.batch import make_batch
from deliverance_b200.models.gpt2 import Gpt2Model
from deliverance_b200.models.transformer import DecoderModel
from deliverance_b200.ops import ref
from deliverance_b200.params import GeneratorParameters

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T", [77, 3000])  # 3000 tokens: the parallel grouping (chunks of 1024 pairs, the last one ragged)
@pytest.mark.parametrize("E,k,mode,renorm", [(8, 2, "softmax_topk", True), (128, 8, "softmax_topk", False), (64, 6, "topk_softmax", False)])
def test_moe_route_gather_combine(E, k, mode, renorm, T):
    H = 256
    g = torch.Generator().manual_seed(E)
    logits = torch.randn(T, E, generator=g)
    w_ref, idx_ref = ref.moe_route(logits, k, mode, renorm)
    e = ops.require_ext()
    w, idx, counts, offsets, perm, pos = e.moe_route(logits.cuda(), k, 0 if mode == "softmax_topk" else 1, renorm)
    assert torch.equal(idx.cpu().long(), idx_ref) and torch.allclose(w.cpu(), w_ref, atol=1e-5)
    assert counts.cpu().tolist() == torch.bincount(idx_ref.flatten(), minlength=E).tolist()
    assert offsets.cpu().tolist() == [0] + torch.cumsum(torch.bincount(idx_ref.flatten(), minlength=E), 0).tolist()
    flat = idx_ref.flatten()
    assert torch.equal(flat[perm.cpu().long()], torch.sort(flat, stable=True).values)
    assert torch.equal(perm.cpu()[pos.cpu().long()], torch.arange(T * k, dtype=torch.int32))
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    if T > 1000:  # the single-CTA grouping gives the same arrays
        e.moe_parallel_sort(False)
        try:
            serial = e.moe_route(logits.cuda(), k, 0 if mode == "softmax_topk" else 1, renorm)
        finally:
            e.moe_parallel_sort(True)
        for ta, tb in zip((w, idx, counts, offsets, perm, pos), serial):
            assert torch.equal(ta, tb)
    xs = e.moe_gather(x.cuda(), perm, k)
    assert torch.equal(xs.cpu(), x[(perm.cpu() // k).long()])
    ys = torch.randn(T * k, H, generator=g).to(torch.bfloat16)
    out = e.moe_combine(ys.cuda(), pos, w, T, k)
    exp = (ys.float()[pos.cpu().long()].reshape(T, k, H) * w_ref.unsqueeze(-1)).sum(1)
    assert ((out.cpu().float() - exp).norm() / exp.norm()).item() < 1e-2


@pytest.mark.parametrize("T,E,k,mode,renorm,e0,ne,bn", [(1, 8, 2, 0, True, 0, 8, 4), (32, 128, 8, 0, False, 0, 128, 8), (64, 128, 8, 0, True, 32, 48, 8),
                                                        (77, 64, 6, 1, False, 0, 64, 16), (128, 8, 2, 0, True, 4, 4, 64), (5, 1000, 16, 0, True, 0, 1000, 4)])
def test_moe_route_in_one_launch_equals_the_separate_kernels(T, E, k, mode, renorm, e0, ne, bn):
    """Decode-size routing (top-k, histogram, offsets, grouping permutation, work list) from the single-CTA kernel: identical to
    moe_route + moe_items, ties between equal logits included."""
    e = ops.require_ext()
    g = torch.Generator().manual_seed(T * 1000 + E)
    logits = torch.randn(T, E, generator=g)
    logits[:, 1] = logits[:, 0]  # a tie in every row: the lower expert index wins in both
    rows = T * k
    max_items = max(1, min((rows + bn - 1) // bn + ne, rows) if rows >= ne else rows)
    a = e.moe_route(logits.cuda(), k, mode, renorm)
    items_a = e.moe_items(a[3], e0, ne, bn, max_items)
    b = e.moe_route_items(logits.cuda(), k, mode, renorm, e0, ne, bn, max_items)
    assert len(b) == 7
    torch.cuda.synchronize()
    for name, ta, tb in zip(("w", "idx", "counts", "offsets", "perm", "pos"), a, b):
        assert torch.equal(ta, tb), name
    assert torch.equal(items_a, b[6])
    assert e.moe_route_items(torch.randn(129, E).cuda(), k, mode, renorm, e0, ne, bn, max_items) == []  # beyond its size: the caller falls back


@pytest.mark.parametrize("q4", [False, True])
@pytest.mark.parametrize("T,E,k,N,K,e0,ne", [(40, 8, 2, 256, 512, 0, 8), (64, 16, 4, 384, 1024, 4, 8), (700, 4, 2, 192, 256, 0, 4), (3, 8, 2, 128, 2048, 6, 2),
                                             (24, 4, 2, 176, 1024, 0, 4)])  # 176 / 16 = 11 row groups: the GEMV's last CTA has an empty one
def test_grouped_gemm_matches_per_expert(T, E, k, N, K, e0, ne, q4):
    """Grouped tcgen05 GEMM over the local experts [e0, e0 + ne) of a routed batch against a per-expert fp32 product."""
    from deliverance_b200.ckpt.jq4 import q4_dequantize, q4_quantize
    from deliverance_b200.ckpt.safetensors_io import Q4Tensor
    from deliverance_b200.ops import GroupedLinearWeight, LinearWeight

    e = ops.require_ext()
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g)
    ws = [torch.randn(N, K, generator=g) * 0.05 for _ in range(ne)]
    lws, dense = [], []
    for w in ws:
        if q4:
            pk, sc = q4_quantize(w)
            dense.append(q4_dequantize(pk, sc))
            lws.append(LinearWeight(Q4Tensor(pk, sc, (N, K))).to("cuda", torch.bfloat16))
        else:
            dense.append(w.to(torch.bfloat16).float())
            lws.append(LinearWeight(w.to(torch.bfloat16)).to("cuda", torch.bfloat16))
    grouped = GroupedLinearWeight(lws)
    w_, idx, counts, offsets, perm, pos = e.moe_route(logits.cuda(), k, 0, True)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    xs = e.moe_gather(x.cuda(), perm, k, offsets, e0, ne)
    off = offsets.cpu().tolist()
    for bn, splits in ((ops.moe_token_tile(T * k * ne // E, ne), 1), (16, 2), (64, 4), (4, 1), (8, 1)):  # 4 / 8: CUDA-core grouped GEMV
        max_items = (T * k + bn - 1) // bn + ne
        items = e.moe_items(offsets, e0, ne, bn, max_items)
        it = items.cpu()
        want_items = [(j, r, off[e0 + j + 1]) for j in range(ne) for r in range(off[e0 + j], off[e0 + j + 1], bn)]
        assert [tuple(v[:3]) for v in it[: len(want_items)].tolist()] == want_items and (it[len(want_items):, 0] == -1).all()
        ys = grouped.run(xs, items, bn, splits)
        torch.cuda.synchronize()
        ops.check_status()
        for j in range(ne):
            lo, hi = off[e0 + j], off[e0 + j + 1]
            if hi == lo:
                continue
            rows = x[(perm.cpu()[lo:hi] // k).long()].float()
            exp = rows @ dense[j].t()
            got = ys[lo:hi].cpu().float()
            assert ((got - exp).norm() / exp.norm().clamp_min(1e-6)).item() < 2e-2, (bn, splits, j)
        if bn <= 8 and q4 and N % 16 == 0:
            # the grouped GEMV with the gated activation in its epilogue: rows [0, N / 2) are the gate, [N / 2, N) the up projection
            hm = grouped.run_gemv_act(xs, items, "silu")
            assert hm is not None and tuple(hm.shape) == (xs.shape[0], N // 2)
            hm_ind = grouped.run_gemv_act(x.cuda(), items, "silu", perm, k)  # token rows read through the permutation: no gather
            torch.cuda.synchronize()
            for j in range(ne):
                lo, hi = off[e0 + j], off[e0 + j + 1]
                assert torch.equal(hm_ind[lo:hi], hm[lo:hi]), ("gemv through perm", bn, j)
            for j in range(ne):
                lo, hi = off[e0 + j], off[e0 + j + 1]
                if hi == lo:
                    continue
                rows = x[(perm.cpu()[lo:hi] // k).long()].float()
                gu = (rows @ dense[j].t()).to(torch.bfloat16).float()
                exp = torch.nn.functional.silu(gu[:, : N // 2]) * gu[:, N // 2:]
                got = hm[lo:hi].cpu().float()
                assert ((got - exp).norm() / exp.norm().clamp_min(1e-6)).item() < 3e-2, ("gemv act", bn, j)


def _pair(tmp_path, family, **over):
    d = str(tmp_path / family)
    if family == "gpt2":
        over = dict(n_embd=256, n_head=4, **over)
    elif family == "granitemoehybrid":
        over = dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, mamba_n_heads=8, mamba_d_head=64, mamba_d_state=64, **over)
    elif family in ("qwen3", "qwen3_moe", "gemma2"):
        over = dict(hidden_size=128, **over)
    else:
        over = dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, **over)
    write_tiny_model(d, family, seed=11, std=0.05, **over)
    cfg = load_config(d)
    cls = Gpt2Model if family == "gpt2" else DecoderModel
    cpu = cls(cfg, "cpu").load(WeightLoader(d))
    gpu = cls(cfg, "cuda:0").load(WeightLoader(d))
    return cfg, cpu, gpu


@pytest.mark.parametrize("family", ["llama", "qwen3", "gemma2", "mixtral", "qwen3_moe", "gpt2", "granitemoehybrid"])
def test_prefill_logits_gpu_vs_cpu(tmp_path, family):
    cfg, cpu, gpu = _pair(tmp_path, family)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(3, 250, (n,), generator=g).tolist() for n in (150, 40)]
    outs = []
    for m in (cpu, gpu):
        eng = Engine(m, EngineConfig(num_pages=64, cuda_graphs=False))
        descr, nxt = [], 1
        for i, t in enumerate(seqs):
            n = (len(t) + 31) // 32
            descr.append({"tokens": t, "start": 0, "pages": list(range(nxt, nxt + n)), "state_slot": i})
            nxt += n
        batch = make_batch(descr, 32, m.device)
        outs.append(m.forward(batch, eng.kv, all_rows=True).float().cpu())
    rel = ((outs[0] - outs[1]).norm() / outs[0].norm()).item()
    assert rel < 3e-2, rel
    agree = (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean().item()
    assert agree > 0.9, agree


@pytest.mark.parametrize("family", ["qwen3", "granitemoehybrid"])
def test_generate_gpu_graphs_vs_eager(tmp_path, family):
    cfg, cpu, gpu = _pair(tmp_path, family)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 250, (n,), generator=g).tolist() for n in (70, 33, 140)]
    res = []
    for graphs in (False, True):
        eng = Engine(gpu, EngineConfig(num_pages=128, cuda_graphs=graphs, max_batch_tokens=96))
        rs = eng.generate_batch(prompts, GeneratorParameters(max_tokens=10))
        res.append([r.token_ids for r in rs])
        ops.check_status(0)
    assert res[0] == res[1]


@pytest.mark.parametrize("family", ["qwen3", "gemma2", "mixtral", "qwen3_moe"])
def test_fused_activation_models_gpu(tmp_path, family, monkeypatch):
    """Models loaded with the interleaved gate|up layout (activation in the GEMM epilogue) against the default layout."""
    d = str(tmp_path / family)
    over = dict(hidden_size=128) if family in ("qwen3", "qwen3_moe", "gemma2") else dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2)
    write_tiny_model(d, family, seed=9, std=0.05, quantize=family in ("qwen3", "qwen3_moe"), **over)
    cfg = load_config(d)
    plain = DecoderModel(cfg, "cuda:0").load(WeightLoader(d))
    monkeypatch.setenv("DLV_FUSED_ACT", "1")
    fused = DecoderModel(cfg, "cuda:0").load(WeightLoader(d))
    assert any(lw.fused_act or lw.fused_act_experts for lw in fused.layers)
    g = torch.Generator().manual_seed(4)
    seqs = [torch.randint(3, 250, (n,), generator=g).tolist() for n in (70, 33, 5)]
    outs = []
    for m in (plain, fused):
        eng = Engine(m, EngineConfig(num_pages=128, cuda_graphs=False))
        descr, nxt = [], 1
        for i, t in enumerate(seqs):
            n = (len(t) + 31) // 32
            descr.append({"tokens": t, "start": 0, "pages": list(range(nxt, nxt + n)), "state_slot": i})
            nxt += n
        outs.append(m.forward(make_batch(descr, 32, m.device), eng.kv, all_rows=True).float().cpu())
        ops.check_status(0)
    # the epilogue applies the activation to fp32 accumulators, the two-kernel path to bf16-rounded ones: logits agree to bf16 noise
    rel = ((outs[0] - outs[1]).norm() / outs[0].norm()).item()
    assert rel < 2e-2, rel
    assert (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean().item() > 0.9
    # and the decode path (small token tiles, CUDA graphs) runs on the interleaved layout
    eng = Engine(fused, EngineConfig(num_pages=128, max_batch_tokens=96))
    rs = eng.generate_batch(seqs, GeneratorParameters(max_tokens=8))
    ops.check_status(0)
    assert all(r.generated_tokens == 8 for r in rs)


@pytest.mark.parametrize("family,over", [("qwen3", dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128)),
                                         ("llama", dict(hidden_size=512, num_attention_heads=4, num_key_value_heads=2))])
def test_fused_rope_models_gpu(tmp_path, family, over, monkeypatch):
    """head_dim 128 models: the q|k|v projection with norm + rotary + KV write in its epilogue (the default on CUDA) against the
    projection followed by the separate kernel: prefill logits of two sequences (one longer than a 256-token tile) and decode."""
    d = str(tmp_path / family)
    write_tiny_model(d, family, seed=13, std=0.05, quantize=True, max_position_embeddings=1024, **over)
    cfg = load_config(d)
    assert cfg.head_dim == 128
    monkeypatch.setenv("DLV_FUSED_ROPE", "0")
    plain = DecoderModel(cfg, "cuda:0").load(WeightLoader(d))
    monkeypatch.setenv("DLV_FUSED_ROPE", "auto")
    fused = DecoderModel(cfg, "cuda:0").load(WeightLoader(d))
    assert fused.fused_rope and not plain.fused_rope
    g = torch.Generator().manual_seed(4)
    seqs = [torch.randint(3, 250, (n,), generator=g).tolist() for n in (540, 33)]
    outs, caches = [], []
    for m in (plain, fused):
        eng = Engine(m, EngineConfig(num_pages=128, cuda_graphs=False))
        descr, nxt = [], 1
        for i, t in enumerate(seqs):
            n = (len(t) + 31) // 32
            descr.append({"tokens": t, "start": 0, "pages": list(range(nxt, nxt + n)), "state_slot": i})
            nxt += n
        outs.append(m.forward(make_batch(descr, 32, m.device), eng.kv, all_rows=True).float().cpu())
        caches.append((eng.kv.k[0].float().cpu(), eng.kv.v[0].float().cpu()))
        ops.check_status(0)
    assert ((caches[0][0] - caches[1][0]).norm() / caches[0][0].norm()).item() < 2e-2
    assert ((caches[0][1] - caches[1][1]).norm() / caches[0][1].norm()).item() < 2e-2
    rel = ((outs[0] - outs[1]).norm() / outs[0].norm()).item()
    assert rel < 2e-2, rel
    res = []
    for m in (plain, fused):
        eng = Engine(m, EngineConfig(num_pages=128, max_batch_tokens=2048))
        res.append([r.token_ids for r in eng.generate_batch(seqs, GeneratorParameters(max_tokens=6))])
    assert [r[0] for r in res[0]] == [r[0] for r in res[1]]
