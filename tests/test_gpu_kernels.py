"""Numerics of every CUDA kernel against the plain PyTorch fp32 statement of the same op (deliverance_b200.ops.ref)."""
import math
import time

import pytest
import torch

from deliverance_b200 import ops
from deliverance_b200.ckpt.jq4 import q4_dequantize, q4_quantize
from deliverance_b200.ckpt.safetensors_io import Q4Tensor
from deliverance_b200.ops import LinearWeight, ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _q4_weight(N, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.05
    p, s = q4_quantize(w)
    return Q4Tensor(p, s, (N, K)), q4_dequantize(p, s)


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("q4", [True, False])
def test_gemv_simt(M, q4):
    N, K = 384, 1024
    qt, wd = _q4_weight(N, K)
    lw = (LinearWeight(qt) if q4 else LinearWeight(wd.to(torch.bfloat16))).to(DEV, torch.bfloat16)
    x = (torch.randn(M, K) * 0.5).to(torch.bfloat16).to(DEV)
    y = ops.linear(x, lw, impl=2)
    wref = wd if q4 else wd.to(torch.bfloat16).float()
    yr = x.float().cpu() @ wref.t()
    assert _rel(y.cpu(), yr) < 1e-2


@pytest.mark.parametrize("M,N,K,splits", [
    (1, 256, 512, 1), (8, 256, 1024, 1), (16, 384, 2560, 0), (17, 128, 256, 1), (64, 512, 2048, 0), (64, 2560, 9728, 0),
    (100, 640, 1216, 1), (128, 256, 4096, 2), (300, 384, 1024, 1), (5, 200, 2560, 4), (33, 1000, 608, 0),
    (64, 256, 4096, 8), (48, 384, 4096, -4), (16, 128, 9728, -16), (7, 256, 2048, 3), (600, 256, 512, 0),
    (64, 19456, 1024, 0), (8, 19712, 1280, 0),  # a few tiles more than SMs: the tail tiles are split over k
])
@pytest.mark.parametrize("q4", [True, False])
def test_gemm_tcgen05(M, N, K, splits, q4):
    qt, wd = _q4_weight(N, K, seed=N + K)
    lw = (LinearWeight(qt) if q4 else LinearWeight(wd.to(torch.bfloat16))).to(DEV, torch.bfloat16)
    x = (torch.randn(M, K) * 0.5).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, device=DEV) if (M % 2 == 0) else None
    lw.bias = bias
    y = ops.linear(x, lw, impl=1, force_splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    wref = wd if q4 else wd.to(torch.bfloat16).float()
    yr = x.float().cpu() @ wref.t()
    if bias is not None:
        yr = yr + bias.cpu()
    assert y.shape == (M, N)
    assert _rel(y.cpu(), yr) < 1.5e-2, f"rel err {_rel(y.cpu(), yr)}"
    # fp32 output path
    y32 = ops.linear(x, lw, out_f32=True, impl=1, force_splits=splits)
    assert y32.dtype == torch.float32 and _rel(y32.cpu(), yr) < 1.5e-2
    # repeated launches reuse the split-K scratch and counters
    y2 = ops.linear(x, lw, impl=1, force_splits=splits)
    assert torch.equal(y, y2)


def test_rmsnorm_and_add():
    T, H = 37, 2560
    x = torch.randn(T, H).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H) * 0.1 + 1).to(torch.bfloat16).to(DEV)
    y = ops.rmsnorm(x, w, 1e-6, 0.0)
    assert _rel(y, ref.rmsnorm(x.float(), w.float(), 1e-6)) < 5e-3
    y1 = ops.rmsnorm(x, w, 1e-6, 1.0)
    assert _rel(y1, ref.rmsnorm(x.float(), w.float(), 1e-6, 1.0)) < 5e-3
    res = torch.randn(T, H).to(torch.bfloat16).to(DEV)
    res_ref = res.clone().float()
    y2 = ops.add_rmsnorm(x, res, w, 1e-6, 0.0, 0.5)
    yr = ref.add_rmsnorm(x.float(), res_ref, w.float(), 1e-6, 0.0, 0.5)
    assert _rel(res, res_ref) < 5e-3 and _rel(y2, yr) < 8e-3


def test_layernorm_act_embedding():
    T, H = 19, 768
    x = torch.randn(T, H).to(torch.bfloat16).to(DEV)
    w = torch.randn(H).to(torch.bfloat16).to(DEV)
    b = torch.randn(H).to(torch.bfloat16).to(DEV)
    assert _rel(ops.layernorm(x, w, b, 1e-5), ref.layernorm(x.float(), w.float(), b.float(), 1e-5)) < 5e-3
    gu = torch.randn(T, 2 * 1024).to(torch.bfloat16).to(DEV)
    for act in ("silu", "gelu_pytorch_tanh", "gelu"):
        assert _rel(ops.act_mul(gu, act), ref.act_mul(gu.float(), act)) < 5e-3
    assert _rel(ops.activation(x, "gelu_new"), ref.act_fn("gelu_new")(x.float())) < 5e-3
    table = torch.randn(500, H).to(torch.bfloat16).to(DEV)
    ids = torch.randint(0, 500, (T,), device=DEV)
    assert _rel(ops.embedding(table, ids, 3.0), table[ids].float() * 3.0) < 5e-3
    pos_t = torch.randn(64, H).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 64, (T,), device=DEV)
    assert _rel(ops.embedding(table, ids, 1.0, pos_t, pos), table[ids].float() + pos_t[pos].float()) < 5e-3


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("qk_norm", [True, False])
def test_rope_kv(D, qk_norm):
    T, H, KV, page, pages = 45, 8, 2, 32, 16
    qkv = torch.randn(T, (H + 2 * KV) * D).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 300, (T,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * page)[:T].to(torch.int64).to(DEV)
    cos, sin = ref.rope_tables(D, 512, 1e6)
    cos, sin = cos.to(DEV), sin.to(DEV)
    qn = (torch.randn(D) * 0.1 + 1).to(torch.bfloat16).to(DEV) if qk_norm else None
    kn = (torch.randn(D) * 0.1 + 1).to(torch.bfloat16).to(DEV) if qk_norm else None
    kc = torch.zeros(pages, KV, page, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    kc_r, vc_r = kc.clone().float(), vc.clone().float()
    q_r = ref.qk_prepare_and_cache(qkv.clone().float(), pos.long(), slots, H, KV, D, None if qn is None else qn.float(),
                                   None if kn is None else kn.float(), 1e-6, 0.0, cos, sin, kc_r, vc_r)
    q = ops.rope_kv(qkv, pos, slots, qn, kn, cos, sin, kc, vc, H, KV, D, 1e-6, 0.0)
    assert _rel(q, q_r.reshape(T, H * D)) < 1e-2
    assert _rel(kc, kc_r) < 1e-2 and _rel(vc, vc_r) < 1e-3


def _paged_setup(ctx_lens, KV, D, page=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((c + page - 1) // page for c in ctx_lens) + 1
    kc = (torch.randn(n_pages, KV, page, D, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(n_pages, KV, page, D, generator=g) * 0.5).to(torch.bfloat16)
    width = max((c + page - 1) // page for c in ctx_lens)
    bt = torch.zeros(len(ctx_lens), width, dtype=torch.int32)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    for i, c in enumerate(ctx_lens):
        n = (c + page - 1) // page
        bt[i, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    return kc, vc, bt


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("D,H,KV", [(128, 32, 8), (64, 32, 4), (256, 16, 8), (128, 8, 8), (128, 14, 2), (64, 32, 2)])
@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("softcap,window", [(0.0, 0), (50.0, 0), (0.0, 48)])
def test_decode_attention(D, H, KV, splits, softcap, window, impl):
    """impl 0 = tensor-core kernel (GQA group as MMA rows), impl 1 = CUDA-core kernel; both against the fp32 reference."""
    if impl == 1 and H // KV > 8:
        pytest.skip("the CUDA-core kernel covers groups of up to 8 heads")
    ctx = [1, 31, 32, 33, 100, 257, 700]
    kc, vc, bt = _paged_setup(ctx, KV, D)
    B = len(ctx)
    q = (torch.randn(B, H * D) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    cl = torch.tensor(ctx, dtype=torch.int32)
    o_ref = ref.paged_attention(q.float().reshape(B, H, D), kc.float(), vc.float(), bt, torch.arange(B), torch.ones(B, dtype=torch.long),
                                cl, scale, softcap, window, True).reshape(B, H * D)
    o = ops.decode_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cl.to(DEV), H, scale, softcap, window, splits, impl)
    assert _rel(o.cpu(), o_ref) < 1e-2


@pytest.mark.parametrize("D,H,KV,splits", [(128, 32, 8, 4), (64, 8, 4, 7), (256, 4, 2, 2), (128, 16, 1, 16)])
def test_decode_attention_merges_splits_in_kernel(D, H, KV, splits):
    """Split-KV decode, opt-in form: the CTA that finishes last for a (sequence, KV head) merges the splits itself. Same result as
    the merge in a second launch, bit-identical from launch to launch (the arrival counters return to zero), splits without keys included."""
    ctx = [1, 17, 64, 100, 257, 700, 1500]
    kc, vc, bt = _paged_setup(ctx, KV, D, seed=5)
    B = len(ctx)
    q = (torch.randn(B, H * D) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    cl = torch.tensor(ctx, dtype=torch.int32)
    o_ref = ref.paged_attention(q.float().reshape(B, H, D), kc.float(), vc.float(), bt, torch.arange(B), torch.ones(B, dtype=torch.long),
                                cl, scale, 0.0, 0, True).reshape(B, H * D)
    args = (q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cl.to(DEV), H, scale, 0.0, 0, splits, 0)
    o_two = ops.decode_attention(*args)
    ops.set_decode_merge_in_kernel(True)
    try:
        outs = [ops.decode_attention(*args) for _ in range(3)]
        torch.cuda.synchronize()
    finally:
        ops.set_decode_merge_in_kernel(False)
    assert _rel(outs[0].cpu(), o_ref) < 1e-2
    assert _rel(outs[0].cpu().float(), o_two.cpu().float()) < 4e-3
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("D,H,KV", [(128, 8, 2), (64, 8, 4), (256, 4, 2)])
@pytest.mark.parametrize("softcap,window", [(0.0, 0), (50.0, 0), (0.0, 40)])
def test_prefill_attention(D, H, KV, softcap, window):
    # (q_len, ctx_len): fresh prompts, a chunk continuing a cached prefix, a single-row sequence
    seqs = [(70, 70), (64, 64), (5, 133), (130, 200), (1, 40)]
    ctx = [c for _, c in seqs]
    kc, vc, bt = _paged_setup(ctx, KV, D, seed=3)
    ql = [q for q, _ in seqs]
    T = sum(ql)
    qs = [sum(ql[:i]) for i in range(len(ql))]
    q = (torch.randn(T, H * D) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    ti = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    o_ref = ref.paged_attention(q.float().reshape(T, H, D), kc.float(), vc.float(), bt, ti(qs), ti(ql), ti(ctx), scale, softcap, window,
                                True).reshape(T, H * D)
    o = ops.prefill_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), ti(qs).to(DEV), ti(ql).to(DEV), ti(ctx).to(DEV), H, scale,
                              softcap, window, True)
    assert _rel(o.cpu(), o_ref) < 1e-2


@pytest.mark.parametrize("D,H,KV,softcap,window", [(128, 8, 2, 0.0, 0), (64, 4, 4, 0.0, 0), (256, 4, 2, 30.0, 0), (128, 4, 1, 0.0, 100), (64, 8, 2, 50.0, 37)])
def test_prefill_attention_tcgen05(D, H, KV, softcap, window):
    """The tcgen05 / TMEM / TMA prefill kernel against the fp32 statement: several key tiles, a chunk continuing a cached prefix,
    ragged tails, GQA, soft-cap and sliding window; pages hold garbage beyond the context end (it must never reach the output)."""
    seqs = [(70, 70), (300, 300), (5, 133), (130, 500), (1, 40), (257, 257)]
    ctx = [c for _, c in seqs]
    kc, vc, bt = _paged_setup(ctx, KV, D, seed=3)
    ql = [q for q, _ in seqs]
    T = sum(ql)
    qs = [sum(ql[:i]) for i in range(len(ql))]
    q = (torch.randn(T, H * D) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    ti = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    o_ref = ref.paged_attention(q.float().reshape(T, H, D), kc.float(), vc.float(), bt, ti(qs), ti(ql), ti(ctx), scale, softcap, window,
                                True).reshape(T, H * D)
    o = ops.prefill_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), ti(qs).to(DEV), ti(ql).to(DEV), ti(ctx).to(DEV), H, scale,
                              softcap, window, True, impl="tc")
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(o.cpu(), o_ref) < 1e-2, _rel(o.cpu(), o_ref)
    o2 = ops.prefill_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), ti(qs).to(DEV), ti(ql).to(DEV), ti(ctx).to(DEV), H, scale,
                               softcap, window, True, impl="mma")
    assert _rel(o.cpu(), o2.cpu()) < 1e-2


def test_argmax_and_logits_post():
    B, V = 5, 151936
    logits = torch.randn(B, V, device=DEV)
    logits[0, 77] = logits[0, 99999] = 50.0  # tie: the first maximum wins
    idx, val = ops.argmax(logits)
    assert idx.tolist() == torch.argmax(logits, dim=-1).tolist() and idx[0].item() == 77
    mask = torch.zeros(B, (V + 31) // 32, dtype=torch.int32, device=DEV)
    allowed = [5, 64, 31, 150000, 1]
    for b, t in enumerate(allowed):
        mask[b, t // 32] = 1 << (t % 32) if t % 32 != 31 else -(1 << 31)
    idx2, _ = ops.argmax(logits, mask)
    assert idx2.tolist() == allowed
    # 64 rows (two-stage path: several CTAs per row) and a short vocabulary (one CTA per row), values included
    for BB, VV in ((64, 151936), (130, 151936), (7, 1000)):
        lg = torch.randn(BB, VV, device=DEV)
        i3, v3 = ops.argmax(lg)
        assert torch.equal(i3, torch.argmax(lg, dim=-1)) and torch.allclose(v3, lg.max(dim=-1).values)
    l2 = logits.clone()
    ops.logits_post(l2, mask, 30.0, 0.5)
    exp = torch.tanh(logits * 0.5 / 30.0) * 30.0
    for b, t in enumerate(allowed):
        assert abs(l2[b, t].item() - exp[b, t].item()) < 1e-4
        assert torch.isinf(l2[b]).sum().item() == V - 1


def test_q4_quantize_bit_exact():
    g = torch.Generator().manual_seed(5)
    w = torch.randn(64, 256, generator=g) * 0.1
    w[3, 32:64] = 0.0
    w[5, 0] = -7.0
    p_ref, s_ref = q4_quantize(w)
    p, s = ops.q4_quantize(w.to(DEV))
    assert torch.equal(p.cpu(), p_ref)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    wb = w.to(torch.bfloat16)
    p_ref, s_ref = q4_quantize(wb)
    p, s = ops.q4_quantize(wb.to(DEV))
    assert torch.equal(p.cpu(), p_ref) and torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    d = ops.require_ext().q4_dequantize(p, s, False)
    assert torch.equal(d.cpu(), q4_dequantize(p_ref, s_ref))


@pytest.mark.parametrize("V,peaked", [(1000, True), (32000, True), (151936, True), (151936, False), (4096, False)])
def test_sample_rows_kernel_matches_sorting_sampler(V, peaked):
    """Histogram-select sampling kernel against the sorting implementation (same uniforms): top-k limits, nucleus, uniform
    picks inside the nucleus, masked (-inf) tokens. Fixed-point weights may move a boundary pick: allow a tiny mismatch rate."""
    from deliverance_b200.engine.sampler import sample_top_k_top_p_batch

    g = torch.Generator().manual_seed(V + int(peaked))
    B = 96
    logits = torch.randn(B, V, generator=g) * (4.0 if peaked else 0.3)
    logits[:, ::7] = float("-inf")  # a guided mask
    logits[3, :] = float("-inf")
    logits[3, 5] = 1.0  # a single allowed token
    temps = torch.tensor([0.5, 0.8, 1.0, 1.3] * (B // 4))
    limits = torch.tensor([V, 50, 1, 1000, V, 7] * (B // 6), dtype=torch.int64).clamp(max=V)
    top_ps = torch.tensor([0.0, 0.1, 0.9, 0.5, 0.99, 0.0, 0.3, 1.0] * (B // 8))
    uniform = torch.tensor([False, False, False, True] * (B // 4))
    us = torch.rand(B, generator=g)
    want = sample_top_k_top_p_batch(logits, temps, limits, top_ps, uniform, us)
    e = ops.require_ext()
    tok, ok = e.sample_rows(logits.to(DEV), (1.0 / temps).to(DEV), limits.to(DEV), top_ps.to(DEV), uniform.to(torch.uint8).to(DEV), us.to(DEV))
    torch.cuda.synchronize()
    tok, ok = tok.cpu(), ok.cpu().bool()
    handled = int(ok.sum())
    assert handled >= (0.6 if peaked else 0.3) * B, handled  # flat rows without top-k may fall into the clamped tail
    agree = (tok[ok] == want[ok]).float().mean().item()
    assert agree >= 0.97, (agree, handled)
    assert tok[3].item() == 5 or not ok[3]
    # every handled pick is an allowed token inside the top-k set of its row
    for i in torch.nonzero(ok).flatten().tolist():
        assert logits[i, tok[i]] != float("-inf")
        kth = torch.topk(logits[i], int(limits[i])).values[-1]
        assert logits[i, tok[i]] >= kth


@pytest.mark.parametrize("M,I,K,q4,act", [(1, 256, 256, True, "silu"), (7, 512, 1024, True, "silu"), (64, 9728, 2560, True, "silu"),
                                           (64, 1216, 2560, True, "silu"), (33, 512, 768, False, "gelu_pytorch_tanh"),
                                           (200, 1024, 512, False, "silu"), (64, 19456, 2560, True, "silu")])
def test_gemm_epilogue_gated_activation(M, I, K, q4, act):
    """linear_act (rows interleaved per 64 outputs, act(gate) * up in the epilogue) against act_mul(linear) in fp32."""
    g = torch.Generator().manual_seed(I + K)
    wg, wu = torch.randn(I, K, generator=g) * 0.05, torch.randn(I, K, generator=g) * 0.05
    if q4:
        pg, sg = q4_quantize(wg)
        pu, su = q4_quantize(wu)
        wg, wu = q4_dequantize(pg, sg), q4_dequantize(pu, su)
        mixed = ops.interleave_gate_up(Q4Tensor(pg, sg, (I, K)), Q4Tensor(pu, su, (I, K)))
    else:
        wg, wu = wg.to(torch.bfloat16).float(), wu.to(torch.bfloat16).float()
        mixed = ops.interleave_gate_up(wg.to(torch.bfloat16), wu.to(torch.bfloat16))
    lw = LinearWeight(mixed).to(DEV, torch.bfloat16)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    y = ops.linear_act(x.to(DEV), lw, act)
    torch.cuda.synchronize()
    ops.check_status()
    yr = ref.act_fn(act)(x.float() @ wg.t()) * (x.float() @ wu.t())
    assert y.shape == (M, I) and _rel(y.cpu(), yr) < 2e-2, _rel(y.cpu(), yr)
    assert torch.equal(y, ops.linear_act(x.to(DEV), lw, act))


@pytest.mark.parametrize("M,H,KV,K,q4,qk_norm,rot_half,bias", [(1, 4, 2, 256, True, True, 64, False), (7, 32, 8, 2560, True, True, 64, False),
                                                                (64, 32, 8, 2560, True, True, 64, False), (64, 4, 1, 2560, True, False, 64, True),
                                                                (200, 8, 2, 512, False, True, 64, True), (33, 4, 4, 4096, False, False, 64, False),
                                                                (529, 32, 8, 2560, True, True, 64, False), (700, 4, 2, 512, False, True, 64, False)])
def test_gemm_epilogue_rope_kv(M, H, KV, K, q4, qk_norm, rot_half, bias):
    """linear_rope_kv against the two separate kernels (projection, then rope_kv) on the same inputs: query heads and the
    written cache rows must agree up to the bf16 rounding of the intermediate tensor."""
    D, page = 128, 32
    g = torch.Generator().manual_seed(M + H)
    N = (H + 2 * KV) * D
    qt, wd = _q4_weight(N, K, seed=N + K)
    lw = (LinearWeight(qt) if q4 else LinearWeight(wd.to(torch.bfloat16))).to(DEV, torch.bfloat16)
    lw.bias = torch.randn(N, generator=g).to(DEV) * 0.1 if bias else None
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 500, (M,), generator=g).to(torch.int32).to(DEV)
    n_pages = (M + page - 1) // page + 2
    perm = torch.randperm(n_pages * page, generator=g)[:M].to(torch.int64).to(DEV)
    cos, sin = ref.rope_tables(D, 512, 10000.0, 1.0, rot_dim=2 * rot_half)
    cos, sin = cos.to(DEV), sin.to(DEV)
    qn = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(DEV) if qk_norm else None
    kn = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(DEV) if qk_norm else None
    caches = [torch.zeros(n_pages, KV, page, D, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    q_ref = ops.rope_kv(ops.linear(x, lw), pos, perm, qn, kn, cos, sin, caches[0], caches[1], H, KV, D, 1e-6, 0.0).clone()
    q = ops.linear_rope_kv(x, lw, pos, perm, qn, kn, cos, sin, caches[2], caches[3], H, KV, D, 1e-6, 0.0)
    torch.cuda.synchronize()
    ops.check_status()
    assert q.shape == (M, H * D) and _rel(q.float().cpu(), q_ref.float().cpu()) < 2e-2
    assert _rel(caches[2].float().cpu(), caches[0].float().cpu()) < 2e-2 and _rel(caches[3].float().cpu(), caches[1].float().cpu()) < 2e-2
    untouched = torch.ones(n_pages * page, dtype=torch.bool)
    untouched[perm.cpu()] = False
    assert caches[2].permute(0, 2, 1, 3).reshape(n_pages * page, -1)[untouched].abs().sum() == 0  # no stray cache rows


def test_bounded_peer_wait_runs_out_and_context_survives():
    """A peer-flag wait that nobody satisfies: the kernel gives up after its limit, records status 2 and returns; nothing
    faults and the same context runs the next kernel normally. The "peer" is a second receive area and flag matrix in this GPU's
    own memory that no kernel ever publishes to (a two-rank layout seen from rank 0 with rank 1 absent)."""
    e = ops.require_ext()
    rows, H, ncta = 4, 256, 256
    slab = rows * H
    recv = [torch.zeros(2 * 2 * slab, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    flags = [torch.zeros(2 * ncta, dtype=torch.int32, device=DEV) for _ in range(2)]
    rounds = torch.zeros(ncta, dtype=torch.int32, device=DEV)
    call = torch.zeros(2, dtype=torch.int32, device=DEV)
    comm = e.TpComm(0, 2, [t.data_ptr() for t in recv], [t.data_ptr() for t in flags], slab, ncta, rounds, call)
    comm.set_wait_limit_ms(2.0)
    ops.check_status()  # clear
    x = torch.randn(rows, H, device=DEV).to(torch.bfloat16)
    out = torch.zeros_like(x)
    t0 = time.perf_counter()
    assert e.oneshot_allreduce(x, comm, out)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    with pytest.raises(RuntimeError, match="peer-flag wait"):
        ops.check_status()
    assert out.float().abs().sum().item() == 0.0  # a CTA whose wait ran out writes no result
    assert flags[1][:rows].tolist() == [1] * rows  # rank 0 did publish to the absent peer
    ops.check_status()  # the status word was consumed
    # the context is intact: an ordinary GEMM on the same device gives the right answer
    qt, wd = _q4_weight(256, 512, seed=1)
    lw = LinearWeight(qt).to(DEV, torch.bfloat16)
    xx = (torch.randn(8, 512) * 0.5).to(torch.bfloat16)
    y = ops.linear(xx.to(DEV), lw)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(y.float().cpu(), xx.float() @ wd.t()) < 2e-2


@pytest.mark.parametrize("M,H,KV,D,hidden,inter,qk_norm,off,act", [
    (1, 4, 2, 128, 512, 1024, True, 0.0, "silu"), (7, 4, 2, 128, 512, 1024, True, 0.0, "silu"),
    (33, 8, 2, 64, 512, 768, False, 1.0, "gelu_pytorch_tanh"), (64, 16, 4, 64, 1024, 1536, False, 0.0, "silu"),
    (64, 32, 8, 128, 2560, 9728, True, 0.0, "silu"), (8, 32, 8, 128, 2560, 9728, True, 0.0, "silu")])
def test_decode_chain_matches_separate_kernels(M, H, KV, D, hidden, inter, qk_norm, off, act):
    """One persistent launch (o_proj -> add + norm -> gate|up -> act * up -> down -> add + norm -> q|k|v -> norm / rotary / KV write)
    against the same steps as separate kernels; every buffer the chain writes is compared, rows beyond M must stay untouched."""
    e = ops.require_ext()
    g = torch.Generator().manual_seed(M + hidden)
    page, R = 32, 64
    eps = 1e-6

    def lin(N, K, seed, bias=False):
        qt, _ = _q4_weight(N, K, seed=seed)
        lw = LinearWeight(qt).to(DEV, torch.bfloat16)
        lw.bias = (torch.randn(N, generator=g) * 0.1).to(DEV) if bias else None
        return lw

    w_o, w_gu, w_dn, w_qkv = lin(hidden, H * D, 1), lin(2 * inter, hidden, 2), lin(hidden, inter, 3), lin((H + 2 * KV) * D, hidden, 4, bias=not qk_norm)

    def nw(n):
        return (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).to(DEV)

    n1, n2 = nw(hidden), nw(hidden)
    qn, kn = (nw(D), nw(D)) if qk_norm else (None, None)
    cos, sin = ref.rope_tables(D, 512, 10000.0, 1.0)
    cos, sin = cos.to(DEV), sin.to(DEV)
    attn = (torch.randn(R, H * D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    res0 = (torch.randn(R, hidden, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 500, (M,), generator=g).to(torch.int32).to(DEV)
    n_pages = 4
    slots = torch.randperm(n_pages * page, generator=g)[:M].to(torch.int64).to(DEV)
    caches = [torch.zeros(n_pages, KV, page, D, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    # ---- separate kernels ----
    res_ref = res0[:M].clone()
    x1 = ops.add_rmsnorm(ops.linear(attn[:M], w_o), res_ref, n1, eps, off, 1.0)
    res_mid = res_ref.clone()
    hh = ops.act_mul(ops.linear(x1, w_gu), act)
    x2 = ops.add_rmsnorm(ops.linear(hh, w_dn), res_ref, n2, eps, off, 1.0)
    q_ref = ops.rope_kv(ops.linear(x2, w_qkv), pos, slots, qn, kn, cos, sin, caches[0], caches[1], H, KV, D, eps, off).clone()
    # ---- one launch ----
    res = res0.clone()
    bx1, bh, bx2, bq = (torch.full((R, n), 7.0, dtype=torch.bfloat16, device=DEV) for n in (hidden, inter, hidden, H * D))
    poison = [torch.full((n,), float("nan"), device=DEV) for n in (1 << 22, 1 << 21, 1 << 20, 1 << 22)]
    del poison  # the chain's workspaces come from the allocator's cache: a slot that is read but never written shows up as NaN
    ch = e.DecodeChain()
    ch.add_op(w_o.handle(), attn, 1, residual=res, norm_w=n1, out=bx1, eps=eps, offset=off)
    ch.add_op(w_gu.handle(), bx1, 2, dep=True, scale_src=0, out=bh, act=act)
    ch.add_op(w_dn.handle(), bh, 1, dep=True, residual=res, norm_w=n2, out=bx2, eps=eps, offset=off)
    ch.add_op(w_qkv.handle(), bx2, 3, dep=True, scale_src=2, bias=w_qkv.bias, out=bq)
    ch.set_qkv(qn, kn, cos, sin, caches[2], caches[3], H, KV, eps, off)
    for rep in range(2):  # the second launch finds the counters the first one left (zero) and gives the same result
        res.copy_(res0)
        ch.run(M, pos, slots)
        torch.cuda.synchronize()
        ops.check_status()
        assert ch.counters().abs().sum().item() == 0
        # the norm stages hand on residual * weight; the row factor is applied behind the next projection
        x1u = (res_mid.float() * (n1.float() + off)).to(torch.bfloat16)
        x2u = (res_ref.float() * (n2.float() + off)).to(torch.bfloat16)
        rels = {"x1": _rel(bx1[:M], x1u), "h": _rel(bh[:M], hh), "residual": _rel(res[:M], res_ref), "x2": _rel(bx2[:M], x2u),
                "q": _rel(bq[:M], q_ref), "k_cache": _rel(caches[2], caches[0]), "v_cache": _rel(caches[3], caches[1])}
        assert all(v < 2e-2 for v in rels.values()), rels
        if M < R:
            assert (bx1[M:] == 7.0).all() and (bh[M:] == 7.0).all() and (bq[M:] == 7.0).all() and torch.equal(res[M:], res0[M:])
    first = bq[:M].clone()
    res.copy_(res0)
    ch.run(M, pos, slots)
    torch.cuda.synchronize()
    assert torch.equal(first, bq[:M])  # fixed summation order: bit-identical repeats


def test_xtc_and_logprob_kernels_match_torch():
    """xtc_rows against the row-by-row torch statement of exclude-top-choice, logprob_rows against logsumexp / topk."""
    from deliverance_b200.engine.sampler import xtc_pick

    e = ops.require_ext()
    g = torch.Generator().manual_seed(5)
    B, V = 9, 5000
    logits = torch.randn(B, V, generator=g) * 3
    logits[2, 77] = 30.0  # one dominant token: nothing else is above the threshold
    logits[4, :] = float("-inf")
    logits[4, 10:14] = torch.tensor([1.0, 1.0, 0.5, 2.0])  # ties above the threshold: the first index wins
    temps = [1.0, 0.7, 1.0, 1.3, 1.0, 1.0, 0.5, 1.0, 1.0]
    thr = [0.001, 0.01, 0.1, 0.0005, 0.1, 0.002, 0.01, 0.5, 0.001]
    fire = [1, 1, 1, 1, 1, 0, 1, 1, 1]
    special = [int(torch.argmax(logits[8]))]  # row 8: the top token is special and is returned as is
    got = e.xtc_rows(logits.to(DEV), torch.tensor([1 / t for t in temps], device=DEV), torch.tensor(thr, device=DEV),
                     torch.tensor(fire, dtype=torch.uint8, device=DEV), torch.tensor(special, dtype=torch.int32, device=DEV)).cpu().tolist()
    for b in range(B):
        want = xtc_pick(logits[b] / temps[b], thr[b], 1.0 if fire[b] else 0.0, 0.5, frozenset(special))
        assert got[b] == (-1 if want is None else want), (b, got[b], want)
    assert got[8] == special[0] and got[5] == -1 and got[4] == 12
    # log-probabilities
    lg = logits.clone()
    lg[4, :] = torch.randn(V, generator=g)
    chosen = torch.randint(0, V, (B,), generator=g)
    lp, ti, tv = e.logprob_rows(lg.to(DEV), chosen.to(DEV), 5)
    lse = torch.logsumexp(lg, dim=-1)
    assert torch.allclose(lp.cpu(), lg.gather(1, chosen.unsqueeze(1)).squeeze(1) - lse, atol=1e-4)
    wv, wi = torch.topk(lg, 5, dim=-1)
    assert torch.equal(ti.cpu(), wi) and torch.allclose(tv.cpu(), wv - lse.unsqueeze(1), atol=1e-4)
    lp0, ti0, _ = e.logprob_rows(lg.to(DEV), chosen.to(DEV), 0)
    assert torch.allclose(lp0.cpu(), lp.cpu()) and ti0.shape == (B, 0)


def test_lora_pool_softmax_turboquant_kernels():
    """The small device kernels off the hot path against their PyTorch statements."""
    from deliverance_b200.embedding import SentenceTransformersPooling as P
    from deliverance_b200.kv.turboquant import MseTurboQuantCodec

    e = ops.require_ext()
    g = torch.Generator().manual_seed(11)
    # LoRA delta
    M, K, N, r = 37, 512, 768, 16
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    A = (torch.randn(r, K, generator=g) * 0.1).to(torch.bfloat16)
    B = (torch.randn(N, r, generator=g) * 0.1).to(torch.bfloat16)
    y0 = (torch.randn(M, N, generator=g)).to(torch.bfloat16)
    y = y0.clone().to(DEV)
    e.lora_delta(x.to(DEV), A.to(DEV), B.to(DEV), y)
    want = y0.float() + (x.float() @ A.float().t()) @ B.float().t()
    assert _rel(y.cpu(), want) < 1e-2
    # pooling
    H = 384
    lens = [5, 1, 40, 17]
    starts = [0, 5, 6, 46]
    h = (torch.randn(sum(lens), H, generator=g)).to(torch.bfloat16)
    modes = {0: P.MEAN, 1: P.MAX, 3: P.CLS, 4: P.LAST_TOKEN, 5: P.MEAN_SQRT_LEN, 6: P.WEIGHTED_MEAN}
    for mode, pool in modes.items():
        for norm in (False, True):
            got = e.pool_rows(h.to(DEV), torch.tensor(starts, dtype=torch.int32, device=DEV), torch.tensor(lens, dtype=torch.int32, device=DEV), mode, norm).cpu()
            for s, (a, n) in enumerate(zip(starts, lens)):
                w = pool.pool(h[a:a + n].float())
                if norm:
                    w = w / w.norm().clamp_min(1e-12)
                assert torch.allclose(got[s], w, atol=2e-3, rtol=1e-3), (mode, norm, s)
    got = e.pool_rows(h.to(DEV), torch.tensor(starts, dtype=torch.int32, device=DEV), torch.tensor(lens, dtype=torch.int32, device=DEV), 2, False).cpu()
    assert torch.allclose(got[2], h[6:46].float().sum(0), atol=1e-2)
    # softmax
    lg = torch.randn(3, 7, generator=g) * 4
    assert torch.allclose(e.softmax_rows(lg.to(DEV)).cpu(), torch.softmax(lg, -1), atol=1e-6)
    # TurboQuant: device codes against the host codec (a coordinate on a bucket edge may differ by the summation order)
    for dim, bits in ((128, 3), (64, 4), (96, 2), (256, 8)):
        codec = MseTurboQuantCodec(dim, bits)
        rows = (torch.randn(50, dim, generator=g) * 2).to(torch.bfloat16)
        host = codec.encode(rows.float())
        dev_enc = codec.encode(rows.to(DEV))
        assert dev_enc.codes.shape == host.codes.shape and torch.allclose(dev_enc.norms, host.norms, rtol=1e-4)
        assert (dev_enc.codes != host.codes).float().mean().item() < 0.01
        back_host = codec.decode(host)
        back_dev = codec.decode(host, torch.float32, DEV).cpu()
        assert torch.allclose(back_dev, back_host, atol=1e-3, rtol=1e-3)
        assert _rel(codec.decode(dev_enc, torch.bfloat16, DEV).cpu(), rows) < (0.6 if bits <= 2 else 0.25)


def test_outputs_stay_inside_their_guard_areas():
    """Bounds checking: every output sits between two 4 KB guard areas; after a sweep over ragged shapes (token counts around the
    tile sizes, ragged prefill, split decode attention, norms, fused activation) no guard byte has changed. The checker itself
    is shown to see a changed byte (written from the host, no kernel misbehaves)."""
    ext = ops.require_ext()
    ops.set_bounds_check(True)
    try:
        g = torch.Generator().manual_seed(2)
        N, K = 384, 256
        w = torch.randn(N, K, generator=g) * 0.05
        p, s = q4_quantize(w)
        lw_q = LinearWeight(Q4Tensor(p, s, (N, K))).to(DEV)
        lw_d = LinearWeight(w.to(torch.bfloat16).to(DEV))
        for M in (1, 5, 17, 63, 65, 129, 257, 529):
            x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
            ops.linear(x, lw_q)
            ops.linear(x, lw_d)
            ops.linear(x, lw_q, out_f32=True)
            ops.linear_act(x, lw_q, "silu")
            wn = torch.ones(K, dtype=torch.bfloat16, device=DEV)
            ops.rmsnorm(x, wn, 1e-6)
            ops.add_rmsnorm(x, x.clone(), wn, 1e-6)
        D, H, KV = 128, 8, 2
        seqs = [(70, 70), (5, 133), (257, 257)]
        ctx = [c for _, c in seqs]
        kc, vc, bt = _paged_setup(ctx, KV, D, seed=5)
        ql = [q for q, _ in seqs]
        T = sum(ql)
        qs = [sum(ql[:i]) for i in range(len(ql))]
        q = (torch.randn(T, H * D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
        ti = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
        for impl in ("tc", "mma"):
            ops.prefill_attention(q, kc.to(DEV), vc.to(DEV), bt.to(DEV), ti(qs), ti(ql), ti(ctx), H, 0.09, 0.0, 0, True, impl=impl)
        B = len(ctx)
        qd = (torch.randn(B, H * D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
        for splits in (1, 4):
            ops.decode_attention(qd, kc.to(DEV), vc.to(DEV), bt.to(DEV), ti(ctx), H, 0.09, 0.0, 0, splits)
        torch.cuda.synchronize()
        ops.check_status()
        ops.check_guards()
        # the checker sees a changed guard byte
        ops.rmsnorm(x, wn, 1e-6)
        ext.poke_last_guard()
        with pytest.raises(RuntimeError, match="wrote outside"):
            ops.check_guards()
    finally:
        ops.set_bounds_check(False)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("q4", [True, False])
def test_linear_prefill_token_tiles(bn, q4):
    """Every token tile the prefill-size GEMM can pick (128 / 256 tokens) against the
    fp32 product, with token counts that end inside a tile."""
    ext = ops.require_ext()
    g = torch.Generator().manual_seed(bn)
    N, K = 640, 1152
    w = torch.randn(N, K, generator=g) * 0.05
    if q4:
        p, s = q4_quantize(w)
        lw, wd = LinearWeight(Q4Tensor(p, s, (N, K))).to(DEV), q4_dequantize(p, s)
    else:
        lw, wd = LinearWeight(w.to(torch.bfloat16).to(DEV)), w.to(torch.bfloat16).float()
    ext.gemm_force_bn(bn)
    try:
        for M in (129, 192, 193, 500, 1024):
            x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
            y = ops.linear(x.to(DEV), lw)
            torch.cuda.synchronize()
            ops.check_status()
            assert _rel(y.cpu().float(), x.float() @ wd.t()) < 1e-2, (bn, M)
    finally:
        ext.gemm_force_bn(0)


@pytest.mark.parametrize("split", [0, 4, 8, 16])
@pytest.mark.parametrize("N,K", [(2560, 4096), (384, 256), (200, 1152), (6144, 2560)])
def test_small_batch_gemv_matches_fp32(N, K, split):
    """1..16 token rows of a JQ4 projection on the mma.sync GEMV: plain (bf16 and fp32 output, bias), gated activation epilogue, and
    agreement with the tcgen05 kernel it replaces at these sizes; every number of K-splitting warps per CTA (0: chosen per shape)."""
    ext = ops.require_ext()
    ext.gemv_force_split(split)
    ops.set_gemv_max_rows(16)  # the two-group form (9..16 rows) is covered too; by default it takes up to 8
    try:
        _small_batch_gemv_case(ext, N, K)
    finally:
        ext.gemv_force_split(0)
        ops.set_gemv_max_rows(8)


def _small_batch_gemv_case(ext, N, K):
    g = torch.Generator().manual_seed(N + K)
    w = torch.randn(N, K, generator=g) * 0.05
    p, s = q4_quantize(w)
    wd = q4_dequantize(p, s)
    bias = torch.randn(N, generator=g) * 0.1
    lw = LinearWeight(Q4Tensor(p, s, (N, K))).to(DEV)
    lwb = LinearWeight(Q4Tensor(p, s, (N, K)), bias=bias).to(DEV)
    for M in (1, 2, 5, 8, 9, 13, 16):
        x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
        ref_y = x.float() @ wd.t()
        assert lw.handle().gemv_ok(M, K) and not lw.handle().gemv_ok(17, K)
        y = ops.linear(x.to(DEV), lw)
        y32 = ops.linear(x.to(DEV), lwb, out_f32=True)
        ext.gemv_dense(False)
        try:
            y_tc = ops.linear(x.to(DEV), lw)
        finally:
            ext.gemv_dense(True)
        torch.cuda.synchronize()
        ops.check_status()
        assert y32.dtype == torch.float32 and _rel(y.cpu().float(), ref_y) < 1e-2 and _rel(y32.cpu(), ref_y + bias) < 1e-2
        assert _rel(y.cpu().float(), y_tc.cpu().float()) < 1e-2
        if N % 32 == 0:
            h = ops.linear_gated(x.to(DEV), lw, "silu")
            gu = ref_y.to(torch.bfloat16).float()
            exp = torch.nn.functional.silu(gu[:, : N // 2]) * gu[:, N // 2:]
            assert tuple(h.shape) == (M, N // 2) and _rel(h.cpu().float(), exp) < 2e-2


@pytest.mark.parametrize("N,K,M", [(640, 1024, 500), (384, 512, 257), (2560, 4096, 2048), (200, 512, 1000)])
def test_persistent_prefill_gemm(N, K, M):
    """The persistent JQ4 GEMM (many tiles per CTA, epilogue under the next tile's main loop) against the fp32 product and against
    the one-tile-per-CTA kernel: bf16 and fp32 output, bias, ragged last token tile and last weight tile."""
    ext = ops.require_ext()
    g = torch.Generator().manual_seed(N + M)
    w = torch.randn(N, K, generator=g) * 0.05
    p, s = q4_quantize(w)
    wd = q4_dequantize(p, s)
    bias = torch.randn(N, generator=g) * 0.1
    lw = LinearWeight(Q4Tensor(p, s, (N, K))).to(DEV)
    lwb = LinearWeight(Q4Tensor(p, s, (N, K)), bias=bias).to(DEV)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    ext.gemm_persist(False)
    try:
        y0 = ops.linear(x.to(DEV), lw)
        ext.gemm_persist(True, True, True)  # issuers in k-block order: repeated launches are bit-identical
        y = ops.linear(x.to(DEV), lw)
        y_again = ops.linear(x.to(DEV), lw)
        y32 = ops.linear(x.to(DEV), lwb, out_f32=True)
        ext.gemm_persist(True, True, False)  # racing issuers: same product up to the accumulation order
        y_race = ops.linear(x.to(DEV), lw)
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        ext.gemm_persist(False)
    assert torch.equal(y, y_again)
    assert _rel(y_race.cpu().float(), y.cpu().float()) < 1e-2
    ref_y = x.float() @ wd.t()
    assert _rel(y.cpu().float(), ref_y) < 1e-2 and _rel(y32.cpu(), ref_y + bias) < 1e-2
    assert _rel(y.cpu().float(), y0.cpu().float()) < 1e-2
