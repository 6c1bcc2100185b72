"""Embeddings and sequence classification.

``embed`` pools the final hidden states of a prompt (AVG / MAX / SUM / MODEL pooling, optional L2 normalisation) and
``classify`` = embed -> linear head -> softmax -> label map (reference: core/.../model/AbstractModel.java:905-998).
Sentence-Transformers pooling modes CLS / MAX / MEAN / MEAN_SQRT_LEN / WEIGHTED_MEAN / LAST_TOKEN and the ``modules.json``
recipe follow core/.../embedding/SentenceTransformersPooling.java:4-150 and SentenceTransformersEmbeddingRecipe.
"""
from __future__ import annotations

import enum
import json
import math
import os
from typing import Optional

import torch

from .ckpt.loader import WeightLoader
from .config import load_config
from .models.bert import BertModel
from .tokenizer.auto import AutoTokenizer


class PoolingType(enum.Enum):
    AVG = "avg"
    MAX = "max"
    SUM = "sum"
    MODEL = "model"


class SentenceTransformersPooling(enum.Enum):
    CLS = "cls"
    MAX = "max"
    MEAN = "mean"
    MEAN_SQRT_LEN = "mean_sqrt_len"
    WEIGHTED_MEAN = "weightedmean"
    LAST_TOKEN = "lasttoken"

    def pool(self, h: torch.Tensor) -> torch.Tensor:
        """h ``[n, hidden]`` fp32 rows of one sequence."""
        n = h.shape[0]
        if self is SentenceTransformersPooling.CLS:
            return h[0]
        if self is SentenceTransformersPooling.MAX:
            return h.max(dim=0).values
        if self is SentenceTransformersPooling.MEAN:
            return h.mean(dim=0)
        if self is SentenceTransformersPooling.MEAN_SQRT_LEN:
            return h.sum(dim=0) / math.sqrt(n)
        if self is SentenceTransformersPooling.WEIGHTED_MEAN:
            w = torch.arange(1, n + 1, dtype=h.dtype, device=h.device).unsqueeze(1)
            return (h * w).sum(dim=0) / w.sum()
        return h[-1]


def recipe_from_model_root(model_dir: str) -> tuple[Optional[SentenceTransformersPooling], bool]:
    """Read ``modules.json`` / ``1_Pooling/config.json``: returns (pooling mode or None, normalize flag)."""
    mj = os.path.join(model_dir, "modules.json")
    if not os.path.exists(mj):
        return None, False
    with open(mj) as f:
        modules = json.load(f)
    mode, normalize = None, False
    for m in modules:
        t = m.get("type", "")
        if t.endswith("Pooling"):
            cp = os.path.join(model_dir, m.get("path", ""), "config.json")
            if os.path.exists(cp):
                with open(cp) as f:
                    pc = json.load(f)
                for key, val in (("pooling_mode_cls_token", SentenceTransformersPooling.CLS),
                                 ("pooling_mode_mean_tokens", SentenceTransformersPooling.MEAN),
                                 ("pooling_mode_max_tokens", SentenceTransformersPooling.MAX),
                                 ("pooling_mode_mean_sqrt_len_tokens", SentenceTransformersPooling.MEAN_SQRT_LEN),
                                 ("pooling_mode_weightedmean_tokens", SentenceTransformersPooling.WEIGHTED_MEAN),
                                 ("pooling_mode_lasttoken", SentenceTransformersPooling.LAST_TOKEN)):
                    if pc.get(key):
                        mode = val
                        break
        elif t.endswith("Normalize"):
            normalize = True
    return mode, normalize


_POOL_MODES = {PoolingType.AVG: 0, PoolingType.MAX: 1, PoolingType.SUM: 2, SentenceTransformersPooling.MEAN: 0, SentenceTransformersPooling.MAX: 1,
               SentenceTransformersPooling.CLS: 3, SentenceTransformersPooling.LAST_TOKEN: 4, SentenceTransformersPooling.MEAN_SQRT_LEN: 5,
               SentenceTransformersPooling.WEIGHTED_MEAN: 6}


def pool_rows(h: torch.Tensor, pooling) -> torch.Tensor:
    if isinstance(pooling, SentenceTransformersPooling):
        return pooling.pool(h)
    if pooling is PoolingType.MAX:
        return h.max(dim=0).values
    if pooling is PoolingType.SUM:
        return h.sum(dim=0)
    return h.mean(dim=0)


class EmbeddingModel:
    """Encoder (bert) or decoder hidden states + pooling."""

    def __init__(self, model, tokenizer, model_dir: str):
        self.model = model
        self.tokenizer = tokenizer
        self.cfg = model.cfg
        self.st_pooling, self.st_normalize = recipe_from_model_root(model_dir)

    def _hidden(self, token_lists: list[list[int]]):
        if isinstance(self.model, BertModel):
            return self.model.encode(token_lists)
        from .engine.engine import Engine, EngineConfig
        from .models.batch import make_batch

        page = 32
        pages_needed = sum((len(t) + page - 1) // page for t in token_lists) + 1
        if getattr(self, "_engine", None) is None or self._engine.kv.num_pages < pages_needed:
            self._engine = Engine(self.model, EngineConfig(num_pages=max(64, pages_needed), cuda_graphs=False))
        seqs, nxt = [], 1
        for toks in token_lists:
            n = (len(toks) + page - 1) // page
            seqs.append({"tokens": toks, "start": 0, "pages": list(range(nxt, nxt + n)), "state_slot": len(seqs)})
            nxt += n
        batch = make_batch(seqs, page, self.model.device)
        return self.model.forward_hidden(batch, self._engine.kv), batch

    def encode_text(self, text: str) -> list[int]:
        ids = self.tokenizer.encode(text, add_special_tokens=isinstance(self.model, BertModel))
        return ids[: self.cfg.max_position_embeddings] or [0]

    def embed_many(self, texts: list[str], pooling=PoolingType.AVG, normalize: Optional[bool] = None) -> torch.Tensor:
        toks = [self.encode_text(t) for t in texts]
        h, batch = self._hidden(toks)
        if pooling is PoolingType.MODEL:
            pooling = self.st_pooling or (SentenceTransformersPooling.CLS if isinstance(self.model, BertModel) else SentenceTransformersPooling.LAST_TOKEN)
            if normalize is None:
                normalize = self.st_normalize
        mode = _POOL_MODES.get(pooling)
        if h.is_cuda and h.dtype == torch.bfloat16 and mode is not None:
            # pooling and the L2 normalisation of every sequence in one kernel (csrc/aux.cu::pool_kernel)
            from . import ops

            lens = torch.tensor(list(batch.q_len_host), dtype=torch.int32, device=h.device)
            ops._count()
            return ops.require_ext().pool_rows(h.contiguous(), batch.q_start.to(torch.int32), lens, mode, bool(normalize))
        hf = h.float()
        out = []
        for s, n in zip(batch.q_start.tolist(), batch.q_len_host):
            out.append(pool_rows(hf[s : s + n], pooling))
        e = torch.stack(out)
        if normalize:
            e = e / e.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        return e

    def embed(self, text: str, pooling=PoolingType.AVG, normalize: Optional[bool] = None) -> list[float]:
        return self.embed_many([text], pooling, normalize)[0].tolist()


class ClassifierModel(EmbeddingModel):
    def classify(self, text: str) -> dict[str, float]:
        if not isinstance(self.model, BertModel) or self.model.classifier is None:
            raise ValueError("model has no classifier head")
        from . import ops

        h, batch = self.model.encode([self.encode_text(text)])
        pooled = self.model.pooled_cls(h, batch)
        logits = ops.linear(pooled.contiguous(), self.model.classifier, out_f32=True)[0]
        if logits.is_cuda:
            ops._count()
            probs = ops.require_ext().softmax_rows(logits.float().unsqueeze(0).contiguous())[0].tolist()
        else:
            probs = torch.softmax(logits.float(), dim=-1).tolist()
        id2label = self.cfg.id2label or {v: k for k, v in self.cfg.label2id.items()}
        return {str(id2label.get(i, i)): p for i, p in enumerate(probs)}


def _load(model_dir: str, device: str = "auto", dtype=None):
    from .api import _device, build_model
    from .parallel.context import SINGLE

    cfg = load_config(model_dir)
    model = build_model(cfg, _device(device), dtype, SINGLE)
    model.load(WeightLoader(model_dir))
    return model, AutoTokenizer.from_pretrained(model_dir)


class AutoModelForEmbeddings:
    @staticmethod
    def from_pretrained(model_dir: str, device: str = "auto", dtype=None) -> EmbeddingModel:
        model, tok = _load(model_dir, device, dtype)
        return EmbeddingModel(model, tok, model_dir)


class AutoModelForSequenceClassification:
    @staticmethod
    def from_pretrained(model_dir: str, device: str = "auto", dtype=None) -> ClassifierModel:
        model, tok = _load(model_dir, device, dtype)
        return ClassifierModel(model, tok, model_dir)
