"""Model graphs on the CPU oracle path against Hugging Face ``transformers`` on tiny random checkpoints with real names."""
import pytest
import torch

from deliverance_b200.ckpt.loader import WeightLoader
from deliverance_b200.ckpt.tiny import write_tiny_model
from deliverance_b200.config import load_config
from deliverance_b200.engine.engine import Engine, EngineConfig
from deliverance_b200.models.gpt2 import Gpt2Model
from deliverance_b200.models.transformer import DecoderModel
from deliverance_b200.params import GeneratorParameters

transformers = pytest.importorskip("transformers")
PROMPT = [3, 17, 45, 99, 120, 7, 8, 9, 10, 11, 200, 201, 33, 34, 35, 36, 37, 38, 39, 40, 41, 50, 51, 52, 60, 61, 62, 63, 64, 65, 66, 67, 68, 69]


def _ours(d, chunk=16, head_quant=None):
    cfg = load_config(d)
    cls = Gpt2Model if cfg.model_type == "gpt2" else DecoderModel
    m = cls(cfg, "cpu").load(WeightLoader(d), head_quant=head_quant)
    return m, Engine(m, EngineConfig(num_pages=64, max_batch_tokens=chunk))


@pytest.mark.parametrize("family", ["llama", "mistral", "qwen2", "qwen3", "gemma2", "gemma3_text", "mixtral", "qwen3_moe", "gpt2", "granitemoehybrid"])
def test_greedy_tokens_match_hf(tmp_path, family):
    d = str(tmp_path / family)
    write_tiny_model(d, family, seed=1, std=0.05)
    _, eng = _ours(d)
    r = eng.generate(PROMPT, GeneratorParameters(max_tokens=6))
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, dtype=torch.float32, attn_implementation="eager").eval()
    with torch.no_grad():
        out = hf.generate(torch.tensor([PROMPT]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert r.token_ids == out[0, len(PROMPT):].tolist()


@pytest.mark.parametrize("family", ["llama", "gemma2", "gemma3_text", "granitemoehybrid"])
def test_prefill_logits_match_hf(tmp_path, family):
    d = str(tmp_path / family)
    write_tiny_model(d, family, seed=2, std=0.05)
    m, eng = _ours(d, chunk=4096)
    from deliverance_b200.models.batch import make_batch
    from deliverance_b200 import ops

    batch = make_batch([{"tokens": PROMPT, "start": 0, "pages": [1, 2], "state_slot": 0}], 32, "cpu")
    logits = m.forward(batch, eng.kv, all_rows=True)
    logits = ops.logits_post(logits.clone(), None, m.cfg.final_softcap, 1.0 / m.cfg.logits_scaling)
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, dtype=torch.float32, attn_implementation="eager").eval()
    with torch.no_grad():
        ref = hf(torch.tensor([PROMPT])).logits[0]
    assert torch.allclose(logits, ref, atol=2e-4, rtol=1e-3)


def test_gemma2_sliding_window_differs_from_global(tmp_path):
    d = str(tmp_path / "g")
    write_tiny_model(d, "gemma2", seed=3, std=0.05, sliding_window=8)
    _, eng = _ours(d)
    r = eng.generate(PROMPT, GeneratorParameters(max_tokens=4))
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, dtype=torch.float32, attn_implementation="eager").eval()
    with torch.no_grad():
        out = hf.generate(torch.tensor([PROMPT]), max_new_tokens=4, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert r.token_ids == out[0, len(PROMPT):].tolist()


def test_quantized_checkpoint_and_head_quant(tmp_path):
    d = str(tmp_path / "q")
    write_tiny_model(d, "qwen3", seed=4, std=0.05, quantize=True)
    m, eng = _ours(d, head_quant="Q4")
    assert m.layers[0].qkv.q4 and m.layers[0].down.q4 and m.lm_head.q4
    r = eng.generate(PROMPT, GeneratorParameters(max_tokens=4))
    assert len(r.token_ids) == 4
    # the same weights dequantised to dense give the same tokens (fp32 oracle over the dequantised weights)
    dense = m.layers[0].qkv.dense()
    assert dense.shape == (m.layers[0].qkv.N, m.layers[0].qkv.K)


def test_layer_trace_hook(tmp_path):
    d = str(tmp_path / "t")
    write_tiny_model(d, "llama", seed=5)
    m, eng = _ours(d)
    seen = []
    m.layer_hook = lambda layer, stage, t: seen.append((layer, stage, tuple(t.shape)))
    eng.generate(PROMPT[:5], GeneratorParameters(max_tokens=1))
    assert (-1, "embed", (5, 64)) in seen and (1, "out", (5, 64)) in seen


def test_gemma3_multimodal_wrapper_config_and_prefix(tmp_path):
    """A gemma3 checkpoint in the multimodal layout (nested text_config with most fields left to defaults, wrapper tensor prefix,
    old-style rope_local_base_freq / sliding_window_pattern) loads as its text tower."""
    import json

    from deliverance_b200.ckpt.safetensors_io import write_safetensors
    from deliverance_b200.ckpt.tiny import build_tensors, tiny_config
    from deliverance_b200.config import parse_config

    full = parse_config({"model_type": "gemma3", "text_config": {"hidden_size": 2560, "intermediate_size": 10240, "num_hidden_layers": 34,
                                                                   "rope_scaling": {"factor": 8.0, "rope_type": "linear"}, "sliding_window": 1024},
                         "eos_token_id": [1, 106]})
    assert (full.num_heads, full.num_kv_heads, full.head_dim, full.vocab_size) == (8, 4, 256, 262208)
    assert full.rope_theta == 1e6 and full.rope_local_theta == 10000.0 and full.rope_factor == 8.0 and full.eos_token_ids == (1, 106)
    assert [full.layer_type(i) for i in range(6)] == ["sliding"] * 5 + ["attention"] and full.window(0) == 1024 and full.window(5) == 0
    text = tiny_config("gemma3_text")
    d = tmp_path / "mm"
    d.mkdir()
    tensors = {("language_model." + k): v for k, v in build_tensors(text, 1, std=0.05).items()}
    write_safetensors(str(d / "model.safetensors"), tensors)
    (d / "config.json").write_text(json.dumps({"model_type": "gemma3", "text_config": {k: v for k, v in text.items() if k != "model_type"}}))
    plain = tmp_path / "plain"
    write_tiny_model(str(plain), "gemma3_text", seed=1, std=0.05)
    a = _ours(str(d))[1].generate(PROMPT, GeneratorParameters(max_tokens=4)).token_ids
    b = _ours(str(plain))[1].generate(PROMPT, GeneratorParameters(max_tokens=4)).token_ids
    assert a == b


@pytest.mark.parametrize("variant", ["base", "shared_kv", "k_eq_v", "moe", "no_ple_softcap"])
def test_gemma4_matches_hf(tmp_path, variant):
    """gemma4 text tower against transformers on random tiny checkpoints written by transformers itself (its own tensor
    names): per-layer head shapes, proportional rotary embedding, per-layer inputs, shared KV layers with double-wide MLPs,
    V = K global layers, the MoE block, final softcap."""
    import json

    from deliverance_b200.api import build_model
    from deliverance_b200.config import parse_config

    over = {"base": {}, "shared_kv": dict(num_kv_shared_layers=3, use_double_wide_mlp=True),
            "k_eq_v": dict(attention_k_eq_v=True, num_global_key_value_heads=1),
            "moe": dict(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32),
            "no_ple_softcap": dict(hidden_size_per_layer_input=0, final_logit_softcapping=30.0)}[variant]
    kw = dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
              head_dim=32, global_head_dim=64, sliding_window=8, max_position_embeddings=256, vocab_size_per_layer_input=256,
              hidden_size_per_layer_input=16, layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2)
    kw.update(over)
    torch.manual_seed(0)
    hf = transformers.Gemma4ForCausalLM(transformers.Gemma4TextConfig(**kw)).eval().float()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.08)
            else:
                p.copy_(1 + 0.1 * torch.randn_like(p))
        for n, b in hf.named_buffers():
            if n.endswith("layer_scalar"):
                b.fill_(0.9)
    d = str(tmp_path / "g4")
    hf.save_pretrained(d, safe_serialization=True)
    cfg = load_config(d)
    assert cfg.model_type == "gemma4_text" and cfg.extra["head_dims"] == [32, 32, 64] * 2
    m = build_model(cfg, "cpu", None, __import__("deliverance_b200.parallel.context", fromlist=["SINGLE"]).SINGLE).load(WeightLoader(d))
    eng = Engine(m, EngineConfig(num_pages=64, max_batch_tokens=16))
    got = eng.generate(PROMPT, GeneratorParameters(max_tokens=6)).token_ids
    with torch.no_grad():
        want = hf.generate(torch.tensor([PROMPT]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(PROMPT):].tolist()
        ref_logits = hf(torch.tensor([PROMPT])).logits[0]
    assert got == want
    from deliverance_b200.models.batch import make_batch

    kv = Engine(m, EngineConfig(num_pages=64, max_batch_tokens=4096)).kv
    lg = m.forward(make_batch([{"tokens": PROMPT, "start": 0, "pages": [1, 2], "state_slot": 0}], 32, "cpu"), kv, all_rows=True)
    if cfg.final_softcap:
        lg = torch.tanh(lg / cfg.final_softcap) * cfg.final_softcap
    assert torch.allclose(lg, ref_logits, atol=3e-4, rtol=1e-3)
    if variant == "shared_kv":
        assert kv.k[3] is kv.k[0] or kv.k[3] is kv.k[1] and kv.k[5] is kv.k[2] and m.layers[4].w["gate_proj"].shape[0] == 256
        nested = parse_config({"model_type": "gemma4", "text_config": json.load(open(d + "/config.json")), "eos_token_id": [1, 106]})
        assert nested.extra["shared_from"] == cfg.extra["shared_from"] == [-1, -1, -1, 1, 1, 2] and nested.eos_token_ids == (1, 106)


@pytest.mark.parametrize("family,quantize", [("llama", False), ("gemma2", False), ("qwen3", True), ("mixtral", False), ("qwen3_moe", True)])
def test_fused_activation_layout_matches_separate_kernels(tmp_path, family, quantize, monkeypatch):
    """Opt-in gate|up layout for the GEMM epilogue activation (rows interleaved per 64 outputs): on the oracle path the model
    must produce the same logits as with the concatenated layout and the separate activation kernel."""
    from deliverance_b200 import ops
    from deliverance_b200.models.batch import make_batch

    d = str(tmp_path / family)
    write_tiny_model(d, family, seed=6, std=0.05, quantize=quantize)
    plain, eng = _ours(d, chunk=4096)
    monkeypatch.setenv("DLV_FUSED_ACT", "1")
    fused, eng2 = _ours(d, chunk=4096)
    moe = family in ("mixtral", "qwen3_moe")
    assert all(lw.fused_act_experts if moe else lw.fused_act for lw in fused.layers) and not any(lw.fused_act or lw.fused_act_experts for lw in plain.layers)
    assert (fused.layers[0].experts_gate_up[0] if moe else fused.layers[0].gate_up).q4 == quantize
    batch = make_batch([{"tokens": PROMPT, "start": 0, "pages": [1, 2], "state_slot": 0}], 32, "cpu")
    a = plain.forward(batch, eng.kv, all_rows=True)
    b = fused.forward(batch, eng2.kv, all_rows=True)
    assert torch.allclose(a, b, atol=1e-5, rtol=1e-5)
    g, u = torch.arange(128.0).reshape(128, 1).repeat(1, 4), -torch.arange(128.0).reshape(128, 1).repeat(1, 4)
    mixed = ops.interleave_gate_up(g, u)
    assert mixed[:64, 0].tolist() == list(range(64)) and mixed[64:128, 0].tolist() == [-float(i) for i in range(64)] and mixed[128, 0] == 64
    assert ops.fused_act_kind("silu") == 1 and ops.fused_act_kind("gelu_pytorch_tanh") == 2 and ops.fused_act_kind("relu") == 0
    with pytest.raises(ValueError):
        ops.interleave_gate_up(torch.zeros(100, 4), torch.zeros(100, 4))


def test_fused_rope_path_composes_the_same_operators(tmp_path, monkeypatch):
    """Opt-in q|k|v epilogue path: on the oracle path it must reproduce the default path exactly (same cache contents, same logits)."""
    from deliverance_b200.models.batch import make_batch

    d = str(tmp_path / "q")
    write_tiny_model(d, "qwen3", seed=8, std=0.05, head_dim=128, hidden_size=128)
    plain, eng = _ours(d, chunk=4096)
    monkeypatch.setenv("DLV_FUSED_ROPE", "1")
    fused, eng2 = _ours(d, chunk=4096)
    assert fused.fused_rope and not plain.fused_rope
    batch = make_batch([{"tokens": PROMPT, "start": 0, "pages": [1, 2], "state_slot": 0}], 32, "cpu")
    a, b = plain.forward(batch, eng.kv, all_rows=True), fused.forward(batch, eng2.kv, all_rows=True)
    assert torch.equal(a, b) and torch.equal(eng.kv.k[1], eng2.kv.k[1]) and torch.equal(eng.kv.v[0], eng2.kv.v[0])
    monkeypatch.setenv("DLV_FUSED_ROPE", "1")
    d64 = str(tmp_path / "l")
    write_tiny_model(d64, "llama", seed=8)
    assert not _ours(d64)[0].fused_rope  # head_dim 16: not eligible


def test_make_batch_long_and_short_sequences():
    """Positions, cache slots and token ids of a batch that mixes prompt chunks (built with tensor ops) and short rows (built from
    lists) against the plain statement, in sequence order."""
    from deliverance_b200.models.batch import make_batch

    page = 32
    seqs = [{"tokens": list(range(100, 700)), "start": 5, "pages": list(range(40, 60))},
            {"tokens": [9, 8, 7], "start": 40, "pages": [300, 301]},
            {"tokens": [1], "start": 0, "pages": [400]},
            {"tokens": list(range(50)), "start": 31, "pages": [7, 3, 5]},
            {"tokens": [4, 4], "start": 63, "pages": [11, 12, 13]}]
    b = make_batch(seqs, page, "cpu")
    pos, slots, toks, starts = [], [], [], []
    for s in seqs:
        starts.append(len(pos))
        for j, tk in enumerate(s["tokens"]):
            p = s["start"] + j
            pos.append(p)
            toks.append(tk)
            slots.append(s["pages"][p // page] * page + p % page)
    assert b.positions.tolist() == pos and b.slots.tolist() == slots and b.token_ids.tolist() == toks
    assert b.positions.dtype == torch.int32 and b.slots.dtype == torch.int64 and b.token_ids.dtype == torch.int32
    assert b.q_start.tolist() == starts and b.q_len.tolist() == [len(s["tokens"]) for s in seqs]
    assert b.ctx_len.tolist() == [s["start"] + len(s["tokens"]) for s in seqs] and not b.is_decode
    assert b.block_tables[0, :20].tolist() == list(range(40, 60)) and b.block_tables[2, 0].item() == 400
    d = make_batch([{"tokens": [7], "start": 100, "pages": list(range(5))} for _ in range(3)], page, "cpu")
    assert d.is_decode and d.slots.tolist() == [3 * page + 4] * 3
