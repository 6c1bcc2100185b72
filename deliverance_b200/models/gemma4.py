"""Gemma-4 text decoder.

What differs from the gemma2 / gemma3 graph (reference: core/.../model/gemma4/Gemma4Model.java, Gemma4Config.java:84-180,
Gemma4PleSupport.java; semantics checked against transformers' ``Gemma4TextModel`` on random tiny checkpoints):

* per-layer attention geometry: sliding layers use ``head_dim`` / ``num_key_value_heads``; full-attention layers use
  ``global_head_dim`` and (with ``attention_k_eq_v``) ``num_global_key_value_heads`` with V = K before the key norm and rotation;
* q and k get a per-head RMSNorm with a learned scale, v a scale-free one; attention scores are not scaled (scale 1);
* sliding layers rotate all of ``head_dim`` with base 10k; full layers rotate only the first ``partial_rotary_factor`` of the
  pairs (``proportional`` rotary embedding), the remaining pairs pass through;
* the last ``num_kv_shared_layers`` layers compute no K / V: they attend over the cache of the last earlier layer of their
  type (their MLP may be twice as wide);
* per-layer inputs: a second embedding table gives every token one small vector per layer, mixed with a projection of the
  token embedding; after the feed-forward each layer gates that vector into the residual stream;
* an optional mixture-of-experts block runs beside the dense MLP (router on the un-normed residual), and every layer ends
  with a learned scalar.

This family runs on the framework's PyTorch operator set (``ops/ref.py``) on any device: the hand-written attention kernels
cover head sizes 64 / 128 / 256, the 512-wide global heads are outside them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ckpt.loader import WeightLoader
from ..ops import ref
from .batch import ForwardBatch
from .transformer import DecoderModel


@dataclass
class G4Layer:
    kind: str = "attention"
    head_dim: int = 0
    n_kv: int = 0
    shared_from: int = -1
    k_eq_v: bool = False
    w: dict = field(default_factory=dict)  # name -> tensor


class Gemma4Model(DecoderModel):
    supports_cuda_graphs = False

    def __init__(self, cfg, device="cpu", dtype=None, tp=None):
        from ..parallel.context import SINGLE

        tp = tp or SINGLE
        if tp.enabled:
            raise ValueError("gemma4 is not sharded for tensor parallelism")
        # the base class checks head_dim against the CUDA kernels; this family does not use them
        self.cfg, self.device, self.tp = cfg, torch.device(device), tp
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.n_heads, self.n_kv = cfg.num_heads, cfg.num_kv_heads
        self.layers: list = []
        self.embed = self.final_norm = self.lm_head = None
        self.cos = self.sin = self.cos_local = self.sin_local = None
        self.layer_hook = None
        self.profiler = None
        self.active_lora = None
        self.shard_head = False
        self.vocab_shard = None
        self._moe_impl = None

    # ------------------------------------------------------------------------------------------------ loading
    def load(self, loader: WeightLoader, head_quant: Optional[str] = None, prefix: str = "model.") -> "Gemma4Model":
        cfg, x = self.cfg, self.cfg.extra
        for alt in (prefix, "model.language_model.", "language_model.model.", "language_model."):
            if loader.has(alt + "embed_tokens.weight"):
                prefix = alt
                break
        d = lambda n: self._dev(loader.load_dense(prefix + n))  # noqa: E731
        self.embed = d("embed_tokens.weight")
        self.ple = None
        if x["ple_hidden"]:
            self.ple = {"table": d("embed_tokens_per_layer.weight"), "proj": d("per_layer_model_projection.weight"),
                        "norm": d("per_layer_projection_norm.weight").reshape(-1)}
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            L = G4Layer(cfg.layer_type(i), x["head_dims"][i], x["kv_heads"][i], x["shared_from"][i], x["k_eq_v"][i])
            w = L.w
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                w[n] = d(p + n + ".weight").reshape(-1)
            w["q"] = d(p + "self_attn.q_proj.weight")
            w["o"] = d(p + "self_attn.o_proj.weight")
            w["q_norm"] = d(p + "self_attn.q_norm.weight").reshape(-1)
            if L.shared_from < 0:
                w["k"] = d(p + "self_attn.k_proj.weight")
                w["k_norm"] = d(p + "self_attn.k_norm.weight").reshape(-1)
                if not L.k_eq_v:
                    w["v"] = d(p + "self_attn.v_proj.weight")
            for n in ("gate_proj", "up_proj", "down_proj"):
                w[n] = d(p + f"mlp.{n}.weight")
            w["layer_scalar"] = d(p + "layer_scalar").reshape(-1) if loader.has(prefix + p + "layer_scalar") else None
            if x["ple_hidden"]:
                w["ple_gate"] = d(p + "per_layer_input_gate.weight")
                w["ple_proj"] = d(p + "per_layer_projection.weight")
                w["ple_norm"] = d(p + "post_per_layer_input_norm.weight").reshape(-1)
            if cfg.num_experts > 0:
                w["router_proj"] = d(p + "router.proj.weight")
                w["router_scale"] = d(p + "router.scale").reshape(-1)
                w["router_expert_scale"] = d(p + "router.per_expert_scale").reshape(-1)
                w["experts_gate_up"] = d(p + "experts.gate_up_proj")  # [E, 2I, hidden]
                w["experts_down"] = d(p + "experts.down_proj")  # [E, hidden, I]
                for n in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                    w[n] = d(p + n + ".weight").reshape(-1)
            self.layers.append(L)
        self.final_norm = d("norm.weight").reshape(-1)
        self.head = self._dev(loader.load_dense("lm_head.weight")) if not cfg.tie_word_embeddings and loader.has("lm_head.weight") else self.embed
        # rotary tables: sliding layers rotate the whole head with the local base; full layers rotate the first fraction of
        # the pairs of the (wider) global head and leave the rest alone (zero angle)
        hd_s = cfg.head_dim
        cos, sin = ref.rope_tables(hd_s, cfg.max_position_embeddings, cfg.rope_local_theta or 10000.0, 1.0)
        self.cos_local, self.sin_local = cos.to(self.device), sin.to(self.device)
        hd_g = max(x["head_dims"])
        angles = int(x["rope_partial"] * hd_g // 2)
        inv = torch.zeros(hd_g // 2, dtype=torch.float64)
        inv[:angles] = 1.0 / (cfg.rope_theta ** (torch.arange(0, 2 * angles, 2, dtype=torch.float64) / hd_g)) / cfg.rope_factor
        ang = torch.arange(cfg.max_position_embeddings, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
        self.cos, self.sin = torch.cos(ang).float().to(self.device), torch.sin(ang).float().to(self.device)
        return self

    # ------------------------------------------------------------------------------------------------ forward
    def _norm(self, t: torch.Tensor, w: Optional[torch.Tensor]) -> torch.Tensor:
        if w is None:  # scale-free variant
            w = torch.ones(t.shape[-1], dtype=torch.float32, device=t.device)
        return ref.rmsnorm(t, w, self.cfg.norm_eps, 0.0)

    def _attention(self, i: int, L: G4Layer, x: torch.Tensor, batch: ForwardBatch, kv) -> torch.Tensor:
        w, T, H, hd = L.w, x.shape[0], self.n_heads, L.head_dim
        pos = batch.positions.long()
        cos, sin = (self.cos_local, self.sin_local) if L.kind == "sliding" else (self.cos, self.sin)
        q = ref.linear_dense(x, w["q"]).reshape(T, H, hd)
        q = ref.apply_rope(self._norm(q, w["q_norm"]), pos, cos, sin)
        k_cache, v_cache = kv.layer(i)  # for a shared layer this is the cache of the layer it borrows from
        if L.shared_from < 0:
            k_raw = ref.linear_dense(x, w["k"]).reshape(T, L.n_kv, hd)
            v = k_raw if L.k_eq_v else ref.linear_dense(x, w["v"]).reshape(T, L.n_kv, hd)
            k = ref.apply_rope(self._norm(k_raw, w["k_norm"]), pos, cos, sin)
            v = self._norm(v, None)
            bs = k_cache.shape[2]
            slots = batch.slots.long()
            blk, off = torch.div(slots, bs, rounding_mode="floor"), slots % bs
            k_cache[blk, :, off, :] = k.to(k_cache.dtype)
            v_cache[blk, :, off, :] = v.to(v_cache.dtype)
        window = self.cfg.sliding_window if L.kind == "sliding" else 0
        a = ref.paged_attention(q.contiguous(), k_cache, v_cache, batch.block_tables, batch.q_start, batch.q_len, batch.ctx_len, 1.0, 0.0,
                                window, causal=not self.cfg.extra["bidirectional"])
        return ref.linear_dense(a.reshape(T, H * hd), w["o"])

    def _mlp(self, L: G4Layer, x: torch.Tensor) -> torch.Tensor:
        act = ref.act_fn(self.cfg.hidden_act)
        return ref.linear_dense(act(ref.linear_dense(x, L.w["gate_proj"]).float()).to(x.dtype) * ref.linear_dense(x, L.w["up_proj"]), L.w["down_proj"])

    def _moe(self, L: G4Layer, residual: torch.Tensor) -> torch.Tensor:
        """Router on the scale-free-normed residual (softmax over all experts, top-k, renormalise, per-expert scale); the experts
        see the residual through their own pre-norm."""
        cfg, w = self.cfg, L.w
        r = self._norm(residual, None).float() * w["router_scale"].float() * cfg.hidden_size ** -0.5
        probs = torch.softmax(r @ w["router_proj"].float().t(), dim=-1)
        top_w, top_i = torch.topk(probs, cfg.experts_per_token, dim=-1)
        top_w = top_w / top_w.sum(dim=-1, keepdim=True) * w["router_expert_scale"].float()[top_i]
        x = self._norm(residual, w["pre_feedforward_layernorm_2"])
        out = torch.zeros_like(x, dtype=torch.float32)
        act = ref.act_fn(cfg.hidden_act)
        for e in top_i.unique().tolist():
            tok, slot = torch.where(top_i == e)
            gate, up = ref.linear_dense(x[tok], w["experts_gate_up"][e]).float().chunk(2, dim=-1)
            y = ref.linear_dense((act(gate) * up).to(x.dtype), w["experts_down"][e]).float()
            out.index_add_(0, tok, y * top_w[tok, slot].unsqueeze(1))
        return out.to(x.dtype)

    def _per_layer_inputs(self, ids: torch.Tensor, emb: torch.Tensor) -> Optional[torch.Tensor]:
        if self.ple is None:
            return None
        cfg, P = self.cfg, self.cfg.extra["ple_hidden"]
        T = ids.shape[0]
        table = (self.ple["table"][ids.long()] * math.sqrt(P)).reshape(T, cfg.num_layers, P)
        proj = (ref.linear_dense(emb, self.ple["proj"]) * cfg.hidden_size ** -0.5).reshape(T, cfg.num_layers, P)
        return (self._norm(proj, self.ple["norm"]) + table) * 2.0 ** -0.5

    def forward_hidden(self, batch: ForwardBatch, kv) -> torch.Tensor:
        cfg = self.cfg
        act = ref.act_fn(cfg.hidden_act)
        h = ref.embedding(self.embed, batch.token_ids, cfg.embedding_multiplier, dtype=self.dtype)
        self._trace(-1, "embed", h)
        pli = self._per_layer_inputs(batch.token_ids, h)
        for i, L in enumerate(self.layers):
            w = L.w
            a = self._attention(i, L, self._norm(h, w["input_layernorm"]), batch, kv)
            h = h + self._norm(a, w["post_attention_layernorm"])
            self._trace(i, "attn", h)
            f = self._mlp(L, self._norm(h, w["pre_feedforward_layernorm"]))
            if cfg.num_experts > 0:
                f = self._norm(f, w["post_feedforward_layernorm_1"]) + self._norm(self._moe(L, h), w["post_feedforward_layernorm_2"])
            h = h + self._norm(f, w["post_feedforward_layernorm"])
            if pli is not None:
                g = act(ref.linear_dense(h, w["ple_gate"]).float()).to(h.dtype) * pli[:, i].to(h.dtype)
                h = h + self._norm(ref.linear_dense(g, w["ple_proj"]), w["ple_norm"])
            if w["layer_scalar"] is not None:
                h = h * w["layer_scalar"].to(h.dtype)
            self._trace(i, "out", h)
        return self._norm(h, self.final_norm)

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        return ref.linear_dense(hidden_rows.float(), self.head.float())

    def greedy_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        return torch.argmax(logits, dim=-1)

    def full_logits(self, logits: torch.Tensor) -> torch.Tensor:
        return logits

    # ------------------------------------------------------------------------------------------------ misc
    def kv_layout(self) -> dict:
        cfg, x = self.cfg, self.cfg.extra
        return {"layers": cfg.num_layers, "kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
                "layer_kinds": [cfg.layer_type(i) for i in range(cfg.num_layers)], "kv_heads_per_layer": list(x["kv_heads"]),
                "head_dim_per_layer": list(x["head_dims"]), "shared_from": list(x["shared_from"])}

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        tensors = [self.embed, self.head, self.final_norm] + ([*self.ple.values()] if self.ple else [])
        for L in self.layers:
            tensors += [t for t in L.w.values() if t is not None]
        for t in tensors:
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n

    def set_lora(self, adapter=None, prefix: str = "model.") -> None:
        if adapter is not None:
            raise ValueError("run-time LoRA is not supported for gemma4")
