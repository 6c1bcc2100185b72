"""``config.json`` parsing into one architecture description shared by every model family.

Field handling follows the reference configs: common llama fields (safetensors/.../Config.java:356-366, only a
linear ``rope_scaling.factor`` is applied), gemma2 (core/.../model/gemma2/Gemma2Config.java:13-46), qwen3
(core/.../model/qwen3/Qwen3Config.java:23-90), qwen3_moe (Qwen3MoeConfig.java:19-23), mixtral (MixtralConfig.java),
gpt2 (Gpt2Config.java), granitemoehybrid (GraniteMoeHybridConfig.java:35-70), bert (BertConfig.java).
``model_type`` dispatch covers the strings of AutoModelForCausaLm.java:522-538 that are in scope.

Divergence kept on purpose: gemma2 ``sliding_window`` / ``query_pre_attn_scalar`` are honoured here (HF semantics);
the reference ignores both and attends globally.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Optional

SUPPORTED_MODEL_TYPES = (
    "llama", "mistral", "mixtral", "gemma2", "gemma3_text", "gemma3", "gemma4_text", "gemma4", "qwen2", "qwen3", "qwen3_moe", "gpt2", "granitemoehybrid", "bert",
)

# transformers' Gemma3TextConfig defaults: hub configs of the multimodal checkpoints leave most text fields out
_GEMMA3_TEXT_DEFAULTS = dict(vocab_size=262208, hidden_size=2304, intermediate_size=9216, num_hidden_layers=26, num_attention_heads=8,
                             num_key_value_heads=4, head_dim=256, max_position_embeddings=131072, rms_norm_eps=1e-6,
                             query_pre_attn_scalar=256, sliding_window=4096, bos_token_id=2, eos_token_id=1, pad_token_id=0)


@dataclass
class ModelConfig:
    model_type: str
    vocab_size: int
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int = 4096
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_factor: float = 1.0
    rope_local_theta: float = 0.0  # gemma3: base of the sliding-window layers' rotary table (0 = same table for every layer)
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: tuple[int, ...] = ()
    pad_token_id: Optional[int] = None
    # attention variants
    qkv_bias: bool = False
    qk_norm: bool = False
    attn_scale: Optional[float] = None  # None -> 1/sqrt(head_dim)
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    sliding_window: int = 0
    layer_types: tuple[str, ...] = ()  # per layer: "attention" | "sliding" | "mamba"
    # norms
    norm_weight_offset: float = 0.0  # gemma: (1 + w)
    post_norms: bool = False  # gemma2: post-attention and post-feedforward norms
    # multipliers (granite)
    embedding_multiplier: float = 1.0
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0
    use_rope: bool = True
    add_bos: bool = True
    # MoE
    num_experts: int = 0
    experts_per_token: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_mode: str = "softmax_topk"  # "softmax_topk" (mixtral/qwen3) | "topk_softmax" (granite)
    decoder_sparse_step: int = 1
    mlp_only_layers: tuple[int, ...] = ()
    shared_intermediate_size: int = 0
    # mamba2 (granite hybrid)
    mamba_n_heads: int = 0
    mamba_n_groups: int = 1
    mamba_d_state: int = 0
    mamba_d_head: int = 0
    mamba_d_conv: int = 4
    mamba_expand: int = 2
    mamba_chunk_size: int = 256
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    # bert / classification
    type_vocab_size: int = 0
    label2id: dict = field(default_factory=dict)
    id2label: dict = field(default_factory=dict)
    raw: dict = field(default_factory=dict, repr=False)
    extra: dict = field(default_factory=dict, repr=False)  # family-specific structure (gemma4: per-layer head shapes, shared KV, ...)

    # ---- derived -------------------------------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def scale(self) -> float:
        return self.attn_scale if self.attn_scale is not None else 1.0 / math.sqrt(self.head_dim)

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else "attention"

    def window(self, i: int) -> int:
        return self.sliding_window if self.layer_type(i) == "sliding" else 0

    def is_sparse_layer(self, i: int) -> bool:
        """qwen3_moe: sparse when not in ``mlp_only_layers`` and ``(i+1) % decoder_sparse_step == 0``."""
        if self.num_experts <= 0:
            return False
        if self.model_type == "qwen3_moe":
            return i not in self.mlp_only_layers and (i + 1) % max(1, self.decoder_sparse_step) == 0
        return True

    @property
    def mamba_intermediate(self) -> int:
        return self.mamba_expand * self.hidden_size

    @property
    def mamba_conv_dim(self) -> int:
        return self.mamba_intermediate + 2 * self.mamba_n_groups * self.mamba_d_state


# transformers' Gemma4TextConfig defaults (hub configs nest the text fields and leave defaults out)
_GEMMA4_TEXT_DEFAULTS = dict(vocab_size=262144, hidden_size=2304, intermediate_size=9216, num_hidden_layers=30, num_attention_heads=8,
                             num_key_value_heads=4, head_dim=256, global_head_dim=512, max_position_embeddings=131072, rms_norm_eps=1e-6,
                             sliding_window=512, vocab_size_per_layer_input=262144, hidden_size_per_layer_input=256, bos_token_id=2,
                             eos_token_id=1, pad_token_id=0, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)


def _parse_gemma4(outer: dict) -> ModelConfig:
    """gemma4 text tower (reference: core/.../model/gemma4/Gemma4Config.java:35-180; semantics of transformers' Gemma4TextModel):
    sliding layers use ``head_dim`` and ``num_key_value_heads``; full-attention layers use ``global_head_dim`` and, with
    ``attention_k_eq_v``, ``num_global_key_value_heads`` with values taken from the keys; the last ``num_kv_shared_layers``
    layers reuse the cache of the last earlier layer of their type; the last layer is always a full-attention layer."""
    d = dict(_GEMMA4_TEXT_DEFAULTS)
    d.update({k: v for k, v in (outer.get("text_config") or outer).items() if v is not None})
    for k in ("eos_token_id", "bos_token_id"):
        if outer.get(k) is not None:
            d[k] = outer[k]
    nl, hd = int(d["num_hidden_layers"]), int(d["head_dim"])
    lt = list(d.get("layer_types") or ["full_attention" if (i + 1) % 6 == 0 else "sliding_attention" for i in range(nl)])
    if lt and lt[-1] != "full_attention":
        lt[-1] = "full_attention"
    ghd = int(d.get("global_head_dim") or hd)
    k_eq_v = bool(d.get("attention_k_eq_v"))
    nkv = int(d.get("num_key_value_heads") or d["num_attention_heads"])
    gkv = int(d.get("num_global_key_value_heads") or nkv) if k_eq_v else nkv
    shared_n = int(d.get("num_kv_shared_layers") or 0)
    first_shared = nl - shared_n
    shared_from = []
    for i in range(nl):
        if shared_n > 0 and i >= first_shared > 0:
            prev = [j for j in range(first_shared) if lt[j] == lt[i]]
            shared_from.append(prev[-1])
        else:
            shared_from.append(-1)
    rp = d.get("rope_parameters") or {}
    full = rp.get("full_attention") or {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1e6}
    loc = rp.get("sliding_attention") or {"rope_type": "default", "rope_theta": 10000.0}
    cfg = ModelConfig(
        model_type="gemma4_text", vocab_size=int(d["vocab_size"]), hidden_size=int(d["hidden_size"]), num_layers=nl,
        num_heads=int(d["num_attention_heads"]), num_kv_heads=nkv, head_dim=hd, intermediate_size=int(d["intermediate_size"]),
        max_position_embeddings=int(d["max_position_embeddings"]), norm_eps=float(d["rms_norm_eps"]), rope_theta=float(full.get("rope_theta", 1e6)),
        rope_factor=float(full.get("factor", 1.0)), rope_local_theta=float(loc.get("rope_theta", 10000.0)),
        hidden_act=d.get("hidden_activation") or "gelu_pytorch_tanh", tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
        bos_token_id=d.get("bos_token_id"), eos_token_ids=_eos(d.get("eos_token_id")), pad_token_id=d.get("pad_token_id"), qk_norm=True,
        attn_scale=1.0, final_softcap=float(d.get("final_logit_softcapping") or 0.0), sliding_window=int(d.get("sliding_window") or 0),
        layer_types=tuple("sliding" if "sliding" in t else "attention" for t in lt), embedding_multiplier=math.sqrt(float(d["hidden_size"])),
        num_experts=int(d.get("num_experts") or 0) if d.get("enable_moe_block") else 0, experts_per_token=int(d.get("top_k_experts") or 0),
        moe_intermediate_size=int(d.get("moe_intermediate_size") or d.get("expert_intermediate_size") or 0), raw=d,
    )
    cfg.extra = {
        "head_dims": [hd if t == "sliding" else ghd for t in cfg.layer_types],
        "kv_heads": [nkv if t == "sliding" else gkv for t in cfg.layer_types],
        "k_eq_v": [k_eq_v and t != "sliding" for t in cfg.layer_types],
        "shared_from": shared_from,
        "double_wide": [bool(d.get("use_double_wide_mlp")) and s >= 0 for s in shared_from],
        "rope_partial": float(full.get("partial_rotary_factor", 1.0)) if full.get("rope_type") == "proportional" else 1.0,
        "ple_hidden": int(d.get("hidden_size_per_layer_input") or 0), "ple_vocab": int(d.get("vocab_size_per_layer_input") or 0),
        "bidirectional": d.get("use_bidirectional_attention") == "all",
    }
    return cfg


def _eos(v: Any) -> tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, (list, tuple)):
        return tuple(int(x) for x in v)
    return (int(v),)


def _rope(d: dict, default_theta: float) -> tuple[float, float]:
    theta = d.get("rope_theta")
    rp = d.get("rope_parameters") or {}
    if theta is None:
        theta = rp.get("rope_theta", default_theta)
    rs = d.get("rope_scaling") or {}
    factor = rs.get("factor", 1.0) if isinstance(rs, dict) and rs.get("rope_type", rs.get("type", "linear")) in ("linear", None) else 1.0
    return float(theta), float(factor or 1.0)


def parse_config(d: dict) -> ModelConfig:
    mt = d.get("model_type")
    if mt not in SUPPORTED_MODEL_TYPES:
        raise ValueError(f"unsupported model_type '{mt}' (supported: {', '.join(SUPPORTED_MODEL_TYPES)})")
    if mt in ("gemma4", "gemma4_text"):
        return _parse_gemma4(d)
    if mt in ("gemma3", "gemma3_text"):
        # the multimodal wrapper nests the language model's fields; only the text tower is served
        outer, d = d, dict(_GEMMA3_TEXT_DEFAULTS)
        d.update({k: v for k, v in (outer.get("text_config") or outer).items() if v is not None or k.endswith("softcapping")})
        for k in ("eos_token_id", "bos_token_id"):
            if outer.get(k) is not None:
                d[k] = outer[k]
        d["model_type"] = mt = "gemma3_text"
    if mt == "gpt2":
        h = d["n_embd"]
        nh = d["n_head"]
        return ModelConfig(
            model_type=mt, vocab_size=d["vocab_size"], hidden_size=h, num_layers=d["n_layer"], num_heads=nh,
            num_kv_heads=nh, head_dim=h // nh, intermediate_size=d.get("n_inner") or 4 * h,
            max_position_embeddings=d.get("n_ctx", d.get("n_positions", 1024)),
            norm_eps=d.get("layer_norm_epsilon", 1e-5), hidden_act=d.get("activation_function", "gelu_new"),
            tie_word_embeddings=True, bos_token_id=d.get("bos_token_id"), eos_token_ids=_eos(d.get("eos_token_id")),
            qkv_bias=True, use_rope=False, add_bos=False, raw=d,
        )
    if mt == "bert":
        h = d["hidden_size"]
        nh = d["num_attention_heads"]
        return ModelConfig(
            model_type=mt, vocab_size=d["vocab_size"], hidden_size=h, num_layers=d["num_hidden_layers"], num_heads=nh,
            num_kv_heads=nh, head_dim=h // nh, intermediate_size=d["intermediate_size"],
            max_position_embeddings=d.get("max_position_embeddings", 512), norm_eps=d.get("layer_norm_eps", 1e-12),
            hidden_act=d.get("hidden_act", "gelu"), pad_token_id=d.get("pad_token_id", 0), qkv_bias=True,
            use_rope=False, add_bos=False, type_vocab_size=d.get("type_vocab_size", 2),
            label2id=d.get("label2id") or {}, id2label={int(k): v for k, v in (d.get("id2label") or {}).items()}, raw=d,
        )
    h = d["hidden_size"]
    nh = d["num_attention_heads"]
    nkv = d.get("num_key_value_heads") or nh
    default_theta = 1e6 if mt in ("qwen3", "qwen3_moe", "mixtral") else 10000.0
    theta, factor = _rope(d, default_theta)
    cfg = ModelConfig(
        model_type=mt, vocab_size=d["vocab_size"], hidden_size=h, num_layers=d["num_hidden_layers"], num_heads=nh,
        num_kv_heads=nkv, head_dim=d.get("head_dim") or h // nh, intermediate_size=d.get("intermediate_size", 0),
        max_position_embeddings=d.get("max_position_embeddings", 4096), norm_eps=d.get("rms_norm_eps", 1e-5),
        rope_theta=theta, rope_factor=factor, hidden_act=d.get("hidden_act") or d.get("hidden_activation") or "silu",
        tie_word_embeddings=bool(d.get("tie_word_embeddings", False)), bos_token_id=d.get("bos_token_id"),
        eos_token_ids=_eos(d.get("eos_token_id")), pad_token_id=d.get("pad_token_id"), raw=d,
    )
    nl = cfg.num_layers
    if mt == "qwen2":
        cfg.qkv_bias = True
    elif mt in ("qwen3", "qwen3_moe"):
        cfg.qk_norm = True
        cfg.qkv_bias = bool(d.get("attention_bias", False))
        if mt == "qwen3_moe":
            cfg.num_experts = d.get("num_experts", 0)
            cfg.experts_per_token = d.get("num_experts_per_tok", 0)
            cfg.moe_intermediate_size = d.get("moe_intermediate_size", 0)
            cfg.norm_topk_prob = bool(d.get("norm_topk_prob", False))
            cfg.decoder_sparse_step = d.get("decoder_sparse_step", 1)
            cfg.mlp_only_layers = tuple(d.get("mlp_only_layers") or ())
    elif mt == "mixtral":
        cfg.num_experts = d.get("num_local_experts", 8)
        cfg.experts_per_token = d.get("num_experts_per_tok", 2)
        cfg.moe_intermediate_size = cfg.intermediate_size
        cfg.norm_topk_prob = True
    elif mt == "gemma2":
        cfg.hidden_act = d.get("hidden_activation") or d.get("hidden_act") or "gelu_pytorch_tanh"
        cfg.attn_softcap = float(d.get("attn_logit_softcapping") or 0.0)
        cfg.final_softcap = float(d.get("final_logit_softcapping") or 0.0)
        cfg.norm_weight_offset = 1.0
        cfg.post_norms = True
        cfg.tie_word_embeddings = True
        # embeddings are scaled by sqrt(hidden) rounded to bf16 (reference Gemma2Model.java:59-61)
        import torch

        cfg.embedding_multiplier = float(torch.tensor(math.sqrt(h), dtype=torch.float32).to(torch.bfloat16).float())
        qpas = d.get("query_pre_attn_scalar")
        if qpas:
            cfg.attn_scale = 1.0 / math.sqrt(float(qpas))
        sw = int(d.get("sliding_window") or 0)
        cfg.sliding_window = sw
        if sw > 0:
            lt = d.get("layer_types")
            if lt:
                cfg.layer_types = tuple("sliding" if "sliding" in t else "attention" for t in lt)
            else:  # HF gemma2: even layers slide, odd layers are global
                cfg.layer_types = tuple("sliding" if i % 2 == 0 else "attention" for i in range(nl))
    elif mt == "gemma3_text":
        # gemma2 block layout (four norms with 1 + w, scaled embeddings, tied head) plus per-head q/k RMSNorm, no attention
        # softcap, five sliding-window layers per global layer, and a separate rotary base for the sliding layers
        # (reference: core/.../model/gemma3/Gemma3Model.java:90-140, Gemma3Config.java; semantics of transformers' Gemma3TextModel)
        import torch

        cfg.hidden_act = d.get("hidden_activation") or d.get("hidden_act") or "gelu_pytorch_tanh"
        cfg.attn_softcap = float(d.get("attn_logit_softcapping") or 0.0)
        cfg.final_softcap = float(d.get("final_logit_softcapping") or 0.0)
        cfg.norm_weight_offset = 1.0
        cfg.post_norms = True
        cfg.qk_norm = True
        cfg.tie_word_embeddings = bool(d.get("tie_word_embeddings", True))
        cfg.embedding_multiplier = float(torch.tensor(math.sqrt(h), dtype=torch.float32).to(torch.bfloat16).float())
        cfg.attn_scale = 1.0 / math.sqrt(float(d.get("query_pre_attn_scalar") or cfg.head_dim))
        cfg.sliding_window = int(d.get("sliding_window") or 0)
        lt = d.get("layer_types")
        if lt:
            cfg.layer_types = tuple("sliding" if "sliding" in t else "attention" for t in lt)
        else:
            pat = int(d.get("sliding_window_pattern") or d.get("_sliding_window_pattern") or 6)
            cfg.layer_types = tuple("attention" if (i + 1) % pat == 0 else "sliding" for i in range(nl))
        if cfg.sliding_window <= 0:
            cfg.layer_types = tuple("attention" for _ in range(nl))
        rp = d.get("rope_parameters") or {}
        if "full_attention" in rp:  # per-layer-type rotary parameters (newer configs)
            full, loc = rp["full_attention"], rp.get("sliding_attention") or {}
            cfg.rope_theta = float(full.get("rope_theta", 1e6))
            cfg.rope_factor = float(full.get("factor", 1.0)) if full.get("rope_type", "default") == "linear" else 1.0
            cfg.rope_local_theta = float(loc.get("rope_theta", 10000.0))
        else:
            cfg.rope_theta = float(d.get("rope_theta") or 1e6)
            cfg.rope_local_theta = float(d.get("rope_local_base_freq") or 10000.0)
    elif mt == "granitemoehybrid":
        cfg.embedding_multiplier = float(d.get("embedding_multiplier", 1.0))
        cfg.residual_multiplier = float(d.get("residual_multiplier", 1.0))
        cfg.logits_scaling = float(d.get("logits_scaling", 1.0))
        am = d.get("attention_multiplier")
        cfg.attn_scale = float(am) if am else None
        cfg.add_bos = False
        cfg.use_rope = d.get("position_embedding_type", "rope") == "rope"
        cfg.shared_intermediate_size = d.get("shared_intermediate_size", 0)
        cfg.num_experts = d.get("num_local_experts", 0) or 0
        cfg.experts_per_token = d.get("num_experts_per_tok", 0) or 0
        cfg.moe_intermediate_size = cfg.intermediate_size
        cfg.router_mode = "topk_softmax"
        lt = d.get("layer_types") or ["attention"] * nl
        cfg.layer_types = tuple("mamba" if t == "mamba" else "attention" for t in lt)
        cfg.mamba_n_heads = d.get("mamba_n_heads", 0)
        cfg.mamba_n_groups = d.get("mamba_n_groups", 1)
        cfg.mamba_d_state = d.get("mamba_d_state", 0)
        cfg.mamba_d_head = d.get("mamba_d_head", 0)
        cfg.mamba_d_conv = d.get("mamba_d_conv", 4)
        cfg.mamba_expand = d.get("mamba_expand", 2)
        cfg.mamba_chunk_size = d.get("mamba_chunk_size", 256)
        cfg.mamba_conv_bias = bool(d.get("mamba_conv_bias", True))
        cfg.mamba_proj_bias = bool(d.get("mamba_proj_bias", False))
    if mt in ("llama", "mistral", "mixtral", "qwen2", "qwen3", "qwen3_moe") and d.get("sliding_window") and d.get("use_sliding_window"):
        # parsed for completeness; the reference always attends fully for these families (Qwen3Config.java:23-90)
        pass
    return cfg


def load_config(model_dir: str) -> ModelConfig:
    with open(os.path.join(model_dir, "config.json")) as f:
        return parse_config(json.load(f))
