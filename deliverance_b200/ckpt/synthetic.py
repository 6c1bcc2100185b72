"""In-memory random-weight "checkpoint" with the loader interface, for benchmarks of full-size shapes.

Tensors are drawn N(0, std) on the target device from a per-tensor seed (so every tensor-parallel rank sees the same
full matrix before slicing its shard) and, when requested, JQ4-quantised with the default policy — the same tensors a
random-init HF directory run through the model quantiser would hold, without writing gigabytes to disk.
"""
from __future__ import annotations

import zlib
from typing import Optional

import torch

from .loader import ShardSpec, shard_dense, shard_q4
from .quantizer import DEFAULT_Q4_FILTER
from .safetensors_io import Q4Tensor, TensorInfo
from .tiny import build_tensors  # noqa: F401  (small models reuse the tiny builder)


def _shapes(cfg: dict) -> dict[str, tuple]:
    """name -> shape for decoder families (llama, mistral, qwen2, qwen3, gemma2, gemma3, mixtral, qwen3_moe)."""
    mt = cfg["model_type"]
    h, L, V = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or h // nh
    I = cfg.get("intermediate_size", 0)
    s: dict[str, tuple] = {"model.embed_tokens.weight": (V, h), "model.norm.weight": (h,)}
    if not cfg.get("tie_word_embeddings", False):
        s["lm_head.weight"] = (V, h)
    for i in range(L):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (h,)
        s[p + "post_attention_layernorm.weight"] = (h,)
        s[p + "self_attn.q_proj.weight"] = (nh * hd, h)
        s[p + "self_attn.k_proj.weight"] = (nkv * hd, h)
        s[p + "self_attn.v_proj.weight"] = (nkv * hd, h)
        s[p + "self_attn.o_proj.weight"] = (h, nh * hd)
        if mt == "qwen2":
            s[p + "self_attn.q_proj.bias"], s[p + "self_attn.k_proj.bias"], s[p + "self_attn.v_proj.bias"] = (nh * hd,), (nkv * hd,), (nkv * hd,)
        if mt in ("qwen3", "qwen3_moe", "gemma3_text"):
            s[p + "self_attn.q_norm.weight"] = (hd,)
            s[p + "self_attn.k_norm.weight"] = (hd,)
        if mt in ("gemma2", "gemma3_text"):
            s[p + "pre_feedforward_layernorm.weight"] = (h,)
            s[p + "post_feedforward_layernorm.weight"] = (h,)
        if mt == "mixtral":
            E = cfg["num_local_experts"]
            s[p + "block_sparse_moe.gate.weight"] = (E, h)
            for e in range(E):
                ep = p + f"block_sparse_moe.experts.{e}."
                s[ep + "w1.weight"], s[ep + "w3.weight"], s[ep + "w2.weight"] = (I, h), (I, h), (h, I)
        elif mt == "qwen3_moe" and (i not in cfg.get("mlp_only_layers", []) and (i + 1) % cfg.get("decoder_sparse_step", 1) == 0):
            E, MI = cfg["num_experts"], cfg["moe_intermediate_size"]
            s[p + "mlp.gate.weight"] = (E, h)
            for e in range(E):
                ep = p + f"mlp.experts.{e}."
                s[ep + "gate_proj.weight"], s[ep + "up_proj.weight"], s[ep + "down_proj.weight"] = (MI, h), (MI, h), (h, MI)
        else:
            s[p + "mlp.gate_proj.weight"], s[p + "mlp.up_proj.weight"], s[p + "mlp.down_proj.weight"] = (I, h), (I, h), (h, I)
    return s


class SyntheticLoader:
    def __init__(self, cfg: dict, seed: int = 0, quantize: bool = False, device="cpu", dtype=torch.bfloat16, std: float = 0.02):
        self.cfg = cfg
        self.seed = seed
        self.quantize = quantize
        self.device = torch.device(device)
        self.dtype = dtype
        self.std = std
        self.shapes = _shapes(cfg)
        self.model_dir = "<synthetic>"

    def names(self):
        return list(self.shapes)

    def has(self, name):
        return name in self.shapes

    def is_q4(self, name):
        return self.quantize and DEFAULT_Q4_FILTER(name) and self.shapes[name][-1] % 32 == 0

    def info(self, name):
        return TensorInfo(name, "Q4" if self.is_q4(name) else "BF16", tuple(self.shapes[name]), 0, 0)

    def majority_dtype(self):
        return "Q4" if self.quantize else "BF16"

    def _gen(self, name):
        shape = self.shapes[name]
        g = torch.Generator(device=self.device).manual_seed((self.seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            base = 0.0 if self.cfg["model_type"] in ("gemma2", "gemma3_text") else 1.0
            return (base + torch.randn(shape, generator=g, device=self.device) * 0.02).to(self.dtype)
        if name.endswith(".gate.weight"):  # routers: wider spread so that top-k choices are well separated
            return (torch.randn(shape, generator=g, device=self.device) * 0.5).to(self.dtype)
        return (torch.randn(shape, generator=g, device=self.device) * self.std).to(self.dtype)

    def load(self, name, shard: Optional[ShardSpec] = None):
        t = self._gen(name)
        if self.is_q4(name):
            from .. import ops

            p, s = ops.q4_quantize(t.float())
            q = Q4Tensor(p, s, tuple(t.shape))
            return shard_q4(q, shard) if shard and shard.size > 1 else q
        return shard_dense(t, shard) if shard and shard.size > 1 else t

    def load_dense(self, name, dtype=torch.float32, shard=None):
        t = self.load(name, shard)
        return t.dequantize(dtype) if isinstance(t, Q4Tensor) else t.to(dtype)

    def close(self):
        pass


QWEN3_4B = dict(model_type="qwen3", vocab_size=151936, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960, rms_norm_eps=1e-6,
                rope_theta=1e6, tie_word_embeddings=True, hidden_act="silu", bos_token_id=151643, eos_token_id=151645)
TINYLLAMA = dict(model_type="llama", vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                 num_attention_heads=32, num_key_value_heads=4, max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=10000.0,
                 tie_word_embeddings=False, hidden_act="silu", bos_token_id=1, eos_token_id=2)
MIXTRAL_8X7B = dict(model_type="mixtral", vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                    num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=32768, rms_norm_eps=1e-5, rope_theta=1e6,
                    num_local_experts=8, num_experts_per_tok=2, tie_word_embeddings=False, hidden_act="silu", bos_token_id=1,
                    eos_token_id=2)
QWEN3_30B_A3B = dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=48,
                     num_attention_heads=32, num_key_value_heads=4, head_dim=128, max_position_embeddings=40960, rms_norm_eps=1e-6,
                     rope_theta=1e6, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
                     decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False, hidden_act="silu", bos_token_id=151643,
                     eos_token_id=151645)
GEMMA2_9B = dict(model_type="gemma2", vocab_size=256000, hidden_size=3584, intermediate_size=14336, num_hidden_layers=42,
                 num_attention_heads=16, num_key_value_heads=8, head_dim=256, max_position_embeddings=8192, rms_norm_eps=1e-6,
                 rope_theta=10000.0, attn_logit_softcapping=50.0, final_logit_softcapping=30.0, sliding_window=4096,
                 query_pre_attn_scalar=256, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True, bos_token_id=2,
                 eos_token_id=1)
GEMMA3_4B = dict(model_type="gemma3_text", vocab_size=262208, hidden_size=2560, intermediate_size=10240, num_hidden_layers=34,
                 num_attention_heads=8, num_key_value_heads=4, head_dim=256, max_position_embeddings=131072, rms_norm_eps=1e-6,
                 rope_theta=1e6, rope_local_base_freq=10000.0, rope_scaling={"factor": 8.0, "rope_type": "linear"}, sliding_window=1024,
                 sliding_window_pattern=6, query_pre_attn_scalar=256, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
                 bos_token_id=2, eos_token_id=1)
SHAPES = {"qwen3-4b": QWEN3_4B, "tinyllama": TINYLLAMA, "mixtral-8x7b": MIXTRAL_8X7B, "qwen3-30b-a3b": QWEN3_30B_A3B,
          "gemma2-9b": GEMMA2_9B, "gemma3-4b": GEMMA3_4B}
