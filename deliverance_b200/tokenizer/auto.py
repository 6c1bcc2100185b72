"""Tokenizer loading (``AutoTokenizer.from_pretrained``) over HF ``tokenizer.json`` / ``tokenizer_config.json``.

Families handled by the reference's ``grace`` module (grace/src/main/java/io/teknek/deliverance/grace/AutoTokenizer.java:49-69,
218-230): byte-level BPE (GPT-2, Qwen2), SentencePiece-style Llama/Gemma BPE, BERT WordPiece. Here the Rust ``tokenizers``
runtime executes ``tokenizer.json`` when it is installed; a small built-in byte-level tokenizer covers checkpoints without a
tokenizer file (synthetic benchmark models, tests). The public surface mirrors ``PreTrainedTokenizerBase``
(PreTrainedTokenizerBase.java:72,81,203): ``encode``, ``decode``, special ids, ``chat_template``.
"""
from __future__ import annotations

import json
import os
from typing import Iterable, Optional


class PreTrainedTokenizer:
    def __init__(self, backend, config: dict, special: dict):
        self._tk = backend
        self.config = config
        self.chat_template: Optional[str] = config.get("chat_template")
        self.bos_token = _tok_str(config.get("bos_token"))
        self.eos_token = _tok_str(config.get("eos_token"))
        self.pad_token = _tok_str(config.get("pad_token"))
        self.unk_token = _tok_str(config.get("unk_token"))
        self.add_bos_token = bool(config.get("add_bos_token", False))
        self._special_ids = set(special.values())
        self._special = special

    # -- ids -------------------------------------------------------------------------------------------------------
    def token_to_id(self, token: Optional[str]) -> Optional[int]:
        if token is None:
            return None
        return self._tk.token_to_id(token)

    @property
    def bos_token_id(self) -> Optional[int]:
        return self.token_to_id(self.bos_token)

    @property
    def eos_token_id(self) -> Optional[int]:
        return self.token_to_id(self.eos_token)

    @property
    def vocab_size(self) -> int:
        return self._tk.get_vocab_size(with_added_tokens=True)

    @property
    def special_ids(self) -> set:
        return set(self._special_ids)

    def is_special(self, token_id: int) -> bool:
        return token_id in self._special_ids

    # -- text ------------------------------------------------------------------------------------------------------
    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return list(self._tk.encode(text, add_special_tokens=add_special_tokens).ids)

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False) -> str:
        return self._tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def id_to_token(self, i: int) -> Optional[str]:
        return self._tk.id_to_token(i)


def _tok_str(v) -> Optional[str]:
    if v is None:
        return None
    if isinstance(v, dict):
        return v.get("content")
    return str(v)


class ByteTokenizer:
    """Fallback: bytes 0..255 map to ids ``offset .. offset+255``; a few named specials sit below the offset."""

    def __init__(self, vocab_size: int = 260, bos: int = 1, eos: int = 2):
        self.offset = 3
        self._vocab = max(vocab_size, self.offset + 256)
        self.names = {"<pad>": 0, "<s>": bos, "</s>": eos}
        self.rev = {v: k for k, v in self.names.items()}

    def token_to_id(self, t):
        return self.names.get(t)

    def id_to_token(self, i):
        if i in self.rev:
            return self.rev[i]
        if self.offset <= i < self.offset + 256:
            return chr(i - self.offset)
        return None

    def get_vocab_size(self, with_added_tokens=True):
        return self._vocab

    def encode(self, text, add_special_tokens=False):
        ids = [b + self.offset for b in text.encode("utf-8")]

        class _E:
            pass

        e = _E()
        e.ids = ids
        return e

    def decode(self, ids, skip_special_tokens=False):
        out = bytearray()
        parts = []
        for i in ids:
            if self.offset <= i < self.offset + 256:
                out.append(i - self.offset)
            elif not skip_special_tokens and i in self.rev:
                parts.append(out.decode("utf-8", errors="replace"))
                out = bytearray()
                parts.append(self.rev[i])
        parts.append(out.decode("utf-8", errors="replace"))
        return "".join(parts)


class AutoTokenizer:
    @staticmethod
    def from_pretrained(model_dir: str) -> PreTrainedTokenizer:
        cfg_path = os.path.join(model_dir, "tokenizer_config.json")
        config: dict = {}
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                config = json.load(f)
        tj = os.path.join(model_dir, "tokenizer.json")
        special: dict = {}
        if os.path.exists(tj):
            from tokenizers import Tokenizer

            tk = Tokenizer.from_file(tj)
            with open(tj) as f:
                raw = json.load(f)
            for a in raw.get("added_tokens", []):
                if a.get("special"):
                    special[a["content"]] = a["id"]
        else:
            vocab = 260
            mc = os.path.join(model_dir, "config.json")
            if os.path.exists(mc):
                with open(mc) as f:
                    vocab = json.load(f).get("vocab_size", 260)
            tk = ByteTokenizer(vocab)
            special = dict(tk.names)
            config.setdefault("bos_token", "<s>")
            config.setdefault("eos_token", "</s>")
        tok = PreTrainedTokenizer(tk, config, special)
        for name in ("bos_token", "eos_token", "pad_token"):
            t = getattr(tok, name)
            i = tok.token_to_id(t) if t else None
            if i is not None:
                tok._special_ids.add(i)
        return tok


class IncrementalDetokenizer:
    """Streams text for a growing id list without splitting multi-byte characters: text is released only up to the last
    position that no longer ends in a replacement character."""

    def __init__(self, tokenizer: PreTrainedTokenizer, skip_special: bool):
        self.tk = tokenizer
        self.skip = skip_special
        self.ids: list[int] = []
        self.prefix = 0  # ids[:prefix] are fully emitted
        self.read = 0
        self.text = ""

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        if self.skip and self.tk.is_special(token_id):
            return ""
        prev = self.tk.decode(self.ids[self.prefix:self.read], skip_special_tokens=self.skip)
        cur = self.tk.decode(self.ids[self.prefix:], skip_special_tokens=self.skip)
        if cur.endswith("�"):
            return ""
        delta = cur[len(prev):] if cur.startswith(prev) else cur
        self.prefix = self.read
        self.read = len(self.ids)
        self.text += delta
        return delta
