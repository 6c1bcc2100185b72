"""Random-weight checkpoints with the real tensor names and shape formulas of every supported family.

Used by the tests (tiny shapes) and by the benchmarks (full benchmark shapes, random-init N(0, 0.02)), mirroring the
reference's "HF-ported" test suites that write a synthetic model directory and load it through the normal loader
(core/src/test/.../model/qwen3/Qwen3HfTextModelPortedTest.java:86-93).
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from .safetensors_io import write_safetensors, write_sharded


def _rand(gen, *shape, std=0.02, dtype=torch.float32):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def tiny_config(model_type: str, **over) -> dict:
    base = dict(
        model_type=model_type, vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0,
        bos_token_id=1, eos_token_id=2, hidden_act="silu", tie_word_embeddings=False,
    )
    if model_type in ("qwen3", "qwen3_moe"):
        base.update(head_dim=64 if "head_dim" not in over else over["head_dim"], rope_theta=1e6, tie_word_embeddings=True)
    if model_type == "qwen3_moe":
        base.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True, decoder_sparse_step=1,
                    mlp_only_layers=[])
    if model_type == "mixtral":
        base.update(num_local_experts=4, num_experts_per_tok=2, rope_theta=1e6)
    if model_type == "gemma2":
        base.update(head_dim=64, attn_logit_softcapping=50.0, final_logit_softcapping=30.0, hidden_activation="gelu_pytorch_tanh",
                    sliding_window=64, query_pre_attn_scalar=64, tie_word_embeddings=True)
    if model_type == "gemma3_text":
        base.update(head_dim=64, hidden_activation="gelu_pytorch_tanh", sliding_window=8, query_pre_attn_scalar=64, tie_word_embeddings=True,
                    num_hidden_layers=3, layer_types=["sliding_attention", "sliding_attention", "full_attention"], rms_norm_eps=1e-6,
                    rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                     "full_attention": {"rope_type": "default", "rope_theta": 1000000.0}})
        base.pop("rope_theta")
    if model_type == "gpt2":
        base = dict(model_type="gpt2", vocab_size=256, n_embd=64, n_head=4, n_layer=2, n_ctx=256, n_positions=256,
                    layer_norm_epsilon=1e-5, bos_token_id=1, eos_token_id=2, activation_function="gelu_new")
    if model_type == "bert":
        base = dict(model_type="bert", vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                    num_attention_heads=4, max_position_embeddings=128, layer_norm_eps=1e-12, hidden_act="gelu", type_vocab_size=2,
                    pad_token_id=0)
    if model_type == "granitemoehybrid":
        base.update(
            layer_types=["mamba", "attention"], embedding_multiplier=12.0, attention_multiplier=0.0156, residual_multiplier=0.22,
            logits_scaling=8.0, shared_intermediate_size=64, num_local_experts=0, num_experts_per_tok=0, position_embedding_type="rope",
            mamba_n_heads=4, mamba_n_groups=1, mamba_d_state=16, mamba_d_head=32, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=32,
            mamba_conv_bias=True, mamba_proj_bias=False, tie_word_embeddings=True,
        )
    base.update(over)
    return base


def build_tensors(cfg: dict, seed: int = 0, dtype=torch.float32, std: float = 0.02) -> dict:
    g = torch.Generator().manual_seed(seed)
    mt = cfg["model_type"]
    R = lambda *s: _rand(g, *s, std=std, dtype=dtype)  # noqa: E731
    ones = lambda n: (torch.ones(n) + torch.randn(n, generator=g) * 0.05).to(dtype)  # noqa: E731
    t: dict = {}
    if mt == "gpt2":
        h, L, V, P = cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"], cfg["n_positions"]
        t["wte.weight"] = R(V, h)
        t["wpe.weight"] = R(P, h)
        for i in range(L):
            p = f"h.{i}."
            t[p + "ln_1.weight"], t[p + "ln_1.bias"] = ones(h), R(h)
            t[p + "attn.c_attn.weight"], t[p + "attn.c_attn.bias"] = R(h, 3 * h), R(3 * h)
            t[p + "attn.c_proj.weight"], t[p + "attn.c_proj.bias"] = R(h, h), R(h)
            t[p + "ln_2.weight"], t[p + "ln_2.bias"] = ones(h), R(h)
            t[p + "mlp.c_fc.weight"], t[p + "mlp.c_fc.bias"] = R(h, 4 * h), R(4 * h)
            t[p + "mlp.c_proj.weight"], t[p + "mlp.c_proj.bias"] = R(4 * h, h), R(h)
        t["ln_f.weight"], t["ln_f.bias"] = ones(h), R(h)
        return t
    if mt == "bert":
        h, L, V, I = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["vocab_size"], cfg["intermediate_size"]
        t["embeddings.word_embeddings.weight"] = R(V, h)
        t["embeddings.position_embeddings.weight"] = R(cfg["max_position_embeddings"], h)
        t["embeddings.token_type_embeddings.weight"] = R(cfg["type_vocab_size"], h)
        t["embeddings.LayerNorm.weight"], t["embeddings.LayerNorm.bias"] = ones(h), R(h)
        for i in range(L):
            p = f"encoder.layer.{i}."
            for n in ("query", "key", "value"):
                t[p + f"attention.self.{n}.weight"], t[p + f"attention.self.{n}.bias"] = R(h, h), R(h)
            t[p + "attention.output.dense.weight"], t[p + "attention.output.dense.bias"] = R(h, h), R(h)
            t[p + "attention.output.LayerNorm.weight"], t[p + "attention.output.LayerNorm.bias"] = ones(h), R(h)
            t[p + "intermediate.dense.weight"], t[p + "intermediate.dense.bias"] = R(I, h), R(I)
            t[p + "output.dense.weight"], t[p + "output.dense.bias"] = R(h, I), R(h)
            t[p + "output.LayerNorm.weight"], t[p + "output.LayerNorm.bias"] = ones(h), R(h)
        t["pooler.dense.weight"], t["pooler.dense.bias"] = R(h, h), R(h)
        nl = len(cfg.get("label2id") or {})
        if nl:
            t["classifier.weight"], t["classifier.bias"] = R(nl, h), R(nl)
        return t
    h, L, V = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or h // nh
    I = cfg.get("intermediate_size", 0)
    t["model.embed_tokens.weight"] = R(V, h)
    for i in range(L):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = ones(h) if mt not in ("gemma2", "gemma3_text") else R(h)
        is_mamba = mt == "granitemoehybrid" and cfg["layer_types"][i] == "mamba"
        if is_mamba:
            H, G, S, dh, K = cfg["mamba_n_heads"], cfg["mamba_n_groups"], cfg["mamba_d_state"], cfg["mamba_d_head"], cfg["mamba_d_conv"]
            inter = cfg["mamba_expand"] * h
            assert inter == H * dh, "mamba_expand * hidden must equal mamba_n_heads * mamba_d_head"
            conv_dim = inter + 2 * G * S
            t[p + "mamba.in_proj.weight"] = R(inter + conv_dim + H, h)
            t[p + "mamba.conv1d.weight"] = _rand(g, conv_dim, 1, K, std=0.2, dtype=dtype)
            t[p + "mamba.conv1d.bias"] = R(conv_dim)
            t[p + "mamba.dt_bias"] = _rand(g, H, std=0.5, dtype=dtype)
            t[p + "mamba.A_log"] = torch.log(torch.rand(H, generator=g) * 3 + 0.5).to(dtype)
            t[p + "mamba.D"] = ones(H)
            t[p + "mamba.norm.weight"] = ones(inter)
            t[p + "mamba.out_proj.weight"] = R(h, inter)
        else:
            t[p + "self_attn.q_proj.weight"] = R(nh * hd, h)
            t[p + "self_attn.k_proj.weight"] = R(nkv * hd, h)
            t[p + "self_attn.v_proj.weight"] = R(nkv * hd, h)
            t[p + "self_attn.o_proj.weight"] = R(h, nh * hd)
            if mt == "qwen2":
                for n, w in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd)):
                    t[p + f"self_attn.{n}_proj.bias"] = R(w)
            if mt in ("qwen3", "qwen3_moe"):
                t[p + "self_attn.q_norm.weight"] = ones(hd)
                t[p + "self_attn.k_norm.weight"] = ones(hd)
            if mt == "gemma3_text":  # stored as w - 1
                t[p + "self_attn.q_norm.weight"] = R(hd)
                t[p + "self_attn.k_norm.weight"] = R(hd)
        t[p + "post_attention_layernorm.weight"] = ones(h) if mt not in ("gemma2", "gemma3_text") else R(h)
        if mt in ("gemma2", "gemma3_text"):
            t[p + "pre_feedforward_layernorm.weight"] = R(h)
            t[p + "post_feedforward_layernorm.weight"] = R(h)
        if mt == "mixtral":
            E = cfg["num_local_experts"]
            t[p + "block_sparse_moe.gate.weight"] = _rand(g, E, h, std=0.5, dtype=dtype)
            for e in range(E):
                ep = p + f"block_sparse_moe.experts.{e}."
                t[ep + "w1.weight"], t[ep + "w3.weight"], t[ep + "w2.weight"] = R(I, h), R(I, h), R(h, I)
        elif mt == "qwen3_moe" and (i not in cfg.get("mlp_only_layers", []) and (i + 1) % cfg.get("decoder_sparse_step", 1) == 0):
            E, MI = cfg["num_experts"], cfg["moe_intermediate_size"]
            t[p + "mlp.gate.weight"] = _rand(g, E, h, std=0.5, dtype=dtype)
            for e in range(E):
                ep = p + f"mlp.experts.{e}."
                t[ep + "gate_proj.weight"], t[ep + "up_proj.weight"], t[ep + "down_proj.weight"] = R(MI, h), R(MI, h), R(h, MI)
        elif mt == "granitemoehybrid":
            S = cfg["shared_intermediate_size"]
            t[p + "shared_mlp.input_linear.weight"] = R(2 * S, h)
            t[p + "shared_mlp.output_linear.weight"] = R(h, S)
            E = cfg.get("num_local_experts", 0)
            if E:
                t[p + "block_sparse_moe.router.layer.weight"] = _rand(g, E, h, std=0.5, dtype=dtype)
                t[p + "block_sparse_moe.input_linear.weight"] = R(E, 2 * I, h)
                t[p + "block_sparse_moe.output_linear.weight"] = R(E, h, I)
        else:
            t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"], t[p + "mlp.down_proj.weight"] = R(I, h), R(I, h), R(h, I)
    t["model.norm.weight"] = ones(h) if mt not in ("gemma2", "gemma3_text") else R(h)
    if not cfg.get("tie_word_embeddings", False):
        t["lm_head.weight"] = R(V, h)
    return t


def write_tiny_model(out_dir: str, model_type: str = "llama", seed: int = 0, dtype=torch.float32, quantize: bool = False,
                     sharded: bool = False, config: Optional[dict] = None, std: float = 0.02, **over) -> dict:
    """Write ``config.json`` + safetensors (optionally JQ4-quantised with the default policy) into ``out_dir``."""
    os.makedirs(out_dir, exist_ok=True)
    cfg = config or tiny_config(model_type, **over)
    tensors = build_tensors(cfg, seed, dtype, std)
    if quantize:
        from .quantizer import DEFAULT_Q4_FILTER, quantize_tensor

        tensors = {k: (quantize_tensor(v) if DEFAULT_Q4_FILTER(k) and v.dim() >= 2 and v.shape[-1] % 32 == 0 else v)
                   for k, v in tensors.items()}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    if sharded:
        write_sharded(out_dir, tensors, max_shard_bytes=256 * 1024)
    else:
        write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return cfg
