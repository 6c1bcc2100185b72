"""GPT-2 decoder: learned positions (``wte`` + ``wpe``), LayerNorm, fused ``c_attn`` in Conv1D layout, GELU MLP, tied head.

Tensor names and transposes follow the reference loader (core/.../model/gpt2/Gpt2Model.java:34-118): ``attn.c_attn.weight`` is
``[in, 3*out]`` (Conv1D) and is transposed to ``[3*out, in]``; ``c_proj`` / ``c_fc`` likewise; every projection has a bias.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ckpt.loader import WeightLoader
from ..ops import LinearWeight
from .batch import ForwardBatch
from .transformer import DecoderModel, LayerWeights


class Gpt2Model(DecoderModel):
    def load(self, loader: WeightLoader, head_quant=None, prefix: str = "") -> "Gpt2Model":
        cfg = self.cfg
        if self.tp.enabled:
            raise ValueError("gpt2 is not sharded for tensor parallelism")
        if not loader.has(prefix + "wte.weight") and loader.has("transformer.wte.weight"):
            prefix = "transformer."
        d = lambda n: self._dev(loader.load_dense(prefix + n))  # noqa: E731
        self.embed = d("wte.weight")
        self.wpe = d("wpe.weight")
        for i in range(cfg.num_layers):
            p = f"h.{i}."
            lw = LayerWeights()
            lw.input_norm = (d(p + "ln_1.weight"), d(p + "ln_1.bias"))
            lw.qkv = self._lin(loader.load_dense(prefix + p + "attn.c_attn.weight").t().contiguous(), loader.load_dense(prefix + p + "attn.c_attn.bias"))
            lw.o = self._lin(loader.load_dense(prefix + p + "attn.c_proj.weight").t().contiguous(), loader.load_dense(prefix + p + "attn.c_proj.bias"))
            lw.pre_ff_norm = (d(p + "ln_2.weight"), d(p + "ln_2.bias"))
            lw.gate_up = self._lin(loader.load_dense(prefix + p + "mlp.c_fc.weight").t().contiguous(), loader.load_dense(prefix + p + "mlp.c_fc.bias"))
            lw.down = self._lin(loader.load_dense(prefix + p + "mlp.c_proj.weight").t().contiguous(), loader.load_dense(prefix + p + "mlp.c_proj.bias"))
            self.layers.append(lw)
        self.final_norm = (d("ln_f.weight"), d("ln_f.bias"))
        self.lm_head = LinearWeight(self.embed) if self.device.type == "cuda" else self._lin(self.embed)
        return self

    def forward_hidden(self, batch: ForwardBatch, kv) -> torch.Tensor:
        cfg = self.cfg
        h = ops.embedding(self.embed, batch.token_ids, 1.0, self.wpe, batch.positions, dtype=self.dtype)
        for i, lw in enumerate(self.layers):
            x = ops.layernorm(h, lw.input_norm[0], lw.input_norm[1], cfg.norm_eps)
            qkv = ops.linear(x, lw.qkv)
            k_cache, v_cache = kv.layer(i)
            q = ops.rope_kv(qkv, batch.positions, batch.slots, None, None, None, None, k_cache, v_cache, self.n_heads, self.n_kv,
                            cfg.head_dim, cfg.norm_eps, 0.0)
            if batch.is_decode:
                a = ops.decode_attention(q, k_cache, v_cache, batch.block_tables, batch.ctx_len, self.n_heads, cfg.scale, 0.0, 0,
                                         batch.decode_splits)
            else:
                a = ops.prefill_attention(q, k_cache, v_cache, batch.block_tables, batch.q_start, batch.q_len, batch.ctx_len,
                                          self.n_heads, cfg.scale, 0.0, 0, True, batch.tile_seq, batch.tile_q0, tiles_for=batch.tiles)
            h = h + ops.linear(a, lw.o)
            self._trace(i, "attn", h)
            x = ops.layernorm(h, lw.pre_ff_norm[0], lw.pre_ff_norm[1], cfg.norm_eps)
            f = ops.linear(ops.activation(ops.linear(x, lw.gate_up), cfg.hidden_act), lw.down)
            h = h + f
            self._trace(i, "out", h)
        return ops.layernorm(h, self.final_norm[0], self.final_norm[1], cfg.norm_eps)
