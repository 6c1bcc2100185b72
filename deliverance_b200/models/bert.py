"""BERT-style encoder for embeddings and sequence classification.

Embeddings = word + position + token-type rows, LayerNorm (the reference's ``gatherRowsAdd`` plan,
tensor/.../operations/TensorOperations.java:181-216); post-LN encoder layers with bidirectional attention
(core/.../generator/BertSelfAttention.java:20-175); optional pooler ``tanh(W h_cls + b)`` and classifier head
(core/.../model/bert/BertModel.java:57-70,150-200,255-290). Tensor names accept an optional ``bert.`` prefix.
Attention runs through the same paged kernels as the decoders (non-causal) over a scratch cache sized for the batch.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..ckpt.loader import WeightLoader
from ..config import ModelConfig
from .batch import ForwardBatch, make_batch


class BertModel:
    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.layers: list[dict] = []
        self.pooler = None
        self.classifier = None

    def _dev(self, t):
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def _lin(self, loader, name):
        from ..ckpt.safetensors_io import Q4Tensor

        w = loader.load(name + ".weight")
        b = loader.load_dense(name + ".bias").reshape(-1) if loader.has(name + ".bias") else None
        lw = ops.LinearWeight(w if isinstance(w, Q4Tensor) else w.to(self.dtype), None if b is None else b.float())
        return lw.to(self.device, self.dtype)

    def load(self, loader: WeightLoader) -> "BertModel":
        pre = "bert." if loader.has("bert.embeddings.word_embeddings.weight") else ""
        d = lambda n: self._dev(loader.load_dense(pre + n).reshape(-1) if n.endswith(("LayerNorm.weight", "LayerNorm.bias")) else loader.load_dense(pre + n))  # noqa: E731
        self.word = d("embeddings.word_embeddings.weight")
        self.pos = d("embeddings.position_embeddings.weight")
        self.typ = d("embeddings.token_type_embeddings.weight")
        self.emb_ln = (d("embeddings.LayerNorm.weight"), d("embeddings.LayerNorm.bias"))
        for i in range(self.cfg.num_layers):
            p = f"{pre}encoder.layer.{i}."
            from .transformer import _cat_weights

            parts = [loader.load(p + f"attention.self.{n}.weight") for n in ("query", "key", "value")]
            bias = torch.cat([loader.load_dense(p + f"attention.self.{n}.bias").reshape(-1) for n in ("query", "key", "value")])
            w = _cat_weights(parts)
            from ..ckpt.safetensors_io import Q4Tensor

            qkv = ops.LinearWeight(w if isinstance(w, Q4Tensor) else w.to(self.dtype), bias.float()).to(self.device, self.dtype)
            self.layers.append({
                "qkv": qkv,
                "o": self._lin(loader, p + "attention.output.dense"),
                "ln1": (self._dev(loader.load_dense(p + "attention.output.LayerNorm.weight").reshape(-1)),
                        self._dev(loader.load_dense(p + "attention.output.LayerNorm.bias").reshape(-1))),
                "up": self._lin(loader, p + "intermediate.dense"),
                "down": self._lin(loader, p + "output.dense"),
                "ln2": (self._dev(loader.load_dense(p + "output.LayerNorm.weight").reshape(-1)),
                        self._dev(loader.load_dense(p + "output.LayerNorm.bias").reshape(-1))),
            })
        if loader.has(pre + "pooler.dense.weight"):
            self.pooler = self._lin(loader, pre + "pooler.dense")
        if loader.has("classifier.weight"):
            self.classifier = self._lin(loader, "classifier")
        return self

    def encode(self, token_lists: list[list[int]], token_types: Optional[list[list[int]]] = None) -> tuple[torch.Tensor, ForwardBatch]:
        """Hidden states ``[T, hidden]`` of a ragged batch of sequences (rows of sequence i = q_start[i] .. +q_len[i])."""
        cfg = self.cfg
        page = 32
        seqs, nxt = [], 1
        for toks in token_lists:
            n = (len(toks) + page - 1) // page
            seqs.append({"tokens": toks, "start": 0, "pages": list(range(nxt, nxt + n))})
            nxt += n
        batch = make_batch(seqs, page, self.device)
        types = None
        if token_types is not None:
            types = torch.tensor([t for ts in token_types for t in ts], dtype=torch.int32, device=self.device)
        kc = torch.zeros(nxt, cfg.num_kv_heads, page, cfg.head_dim, dtype=self.dtype, device=self.device)
        vc = torch.zeros_like(kc)
        h = ops.embedding(self.word, batch.token_ids, 1.0, self.pos, batch.positions, self.typ, types, dtype=self.dtype)
        h = ops.layernorm(h, self.emb_ln[0], self.emb_ln[1], cfg.norm_eps)
        for lw in self.layers:
            qkv = ops.linear(h, lw["qkv"])
            q = ops.rope_kv(qkv, batch.positions, batch.slots, None, None, None, None, kc, vc, cfg.num_heads, cfg.num_kv_heads,
                            cfg.head_dim, cfg.norm_eps, 0.0)
            a = ops.prefill_attention(q, kc, vc, batch.block_tables, batch.q_start, batch.q_len, batch.ctx_len, cfg.num_heads,
                                      cfg.scale, 0.0, 0, False, batch.tile_seq, batch.tile_q0, tiles_for=batch.tiles)
            h = ops.layernorm(h + ops.linear(a, lw["o"]), lw["ln1"][0], lw["ln1"][1], cfg.norm_eps)
            f = ops.linear(ops.activation(ops.linear(h, lw["up"]), cfg.hidden_act), lw["down"])
            h = ops.layernorm(h + f, lw["ln2"][0], lw["ln2"][1], cfg.norm_eps)
        return h, batch

    def pooled_cls(self, h: torch.Tensor, batch: ForwardBatch) -> torch.Tensor:
        cls = h.index_select(0, batch.q_start.long())
        if self.pooler is not None:
            cls = torch.tanh(ops.linear(cls.contiguous(), self.pooler).float()).to(h.dtype)
        return cls
