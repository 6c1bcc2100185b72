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


class SentencePieceBackend:
    """``tokenizer.model`` (SentencePiece) behind the backend interface of the ``tokenizers`` runtime."""

    def __init__(self, path: str):
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=path)

    def token_to_id(self, t):
        i = self.sp.piece_to_id(t)
        return i if self.sp.id_to_piece(i) == t else None

    def id_to_token(self, i):
        return self.sp.id_to_piece(int(i)) if 0 <= int(i) < self.sp.get_piece_size() else None

    def get_vocab_size(self, with_added_tokens=True):
        return self.sp.get_piece_size()

    def encode(self, text, add_special_tokens=False):
        ids = self.sp.encode(text)
        if add_special_tokens and self.sp.bos_id() >= 0:
            ids = [self.sp.bos_id()] + ids

        class _E:
            pass

        e = _E()
        e.ids = ids
        return e

    def decode(self, ids, skip_special_tokens=False):
        ids = [int(i) for i in ids]
        if skip_special_tokens:
            ids = [i for i in ids if not self.sp.is_control(i)]
            return self.sp.decode(ids)
        out, run = [], []
        for i in ids:  # control pieces (<s>, </s>) are dropped by the library's decode: spell them out
            if self.sp.is_control(i):
                out.append(self.sp.decode(run))
                out.append(self.sp.id_to_piece(i))
                run = []
            else:
                run.append(i)
        out.append(self.sp.decode(run))
        return "".join(out)


def _legacy_backend(model_dir: str, config: dict):
    """Tokenizer files older than ``tokenizer.json``: SentencePiece ``tokenizer.model`` (llama / mistral / gemma families),
    ``vocab.json`` + ``merges.txt`` (byte-level BPE: gpt2, qwen2), ``vocab.txt`` (BERT WordPiece). Returns (backend, specials)
    or None (reference families: grace/.../AutoTokenizer.java:49-69, 218-230)."""
    p = lambda n: os.path.join(model_dir, n)  # noqa: E731
    if os.path.exists(p("tokenizer.model")):
        tk = SentencePieceBackend(p("tokenizer.model"))
        special = {tk.sp.id_to_piece(i): i for i in range(tk.sp.get_piece_size()) if tk.sp.is_control(i)}
        if tk.sp.bos_id() >= 0:
            config.setdefault("bos_token", tk.sp.id_to_piece(tk.sp.bos_id()))
        if tk.sp.eos_id() >= 0:
            config.setdefault("eos_token", tk.sp.id_to_piece(tk.sp.eos_id()))
        return tk, special
    if os.path.exists(p("vocab.json")) and os.path.exists(p("merges.txt")):
        from tokenizers import Tokenizer, decoders, models, pre_tokenizers

        tk = Tokenizer(models.BPE.from_file(p("vocab.json"), p("merges.txt")))
        tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=bool(config.get("add_prefix_space", False)))
        tk.decoder = decoders.ByteLevel()
        special = {}
        for name in ("bos_token", "eos_token", "unk_token", "pad_token"):
            t = _tok_str(config.get(name)) or ("<|endoftext|>" if name != "pad_token" else None)
            if t and tk.token_to_id(t) is not None:
                special[t] = tk.token_to_id(t)
                config.setdefault(name, t)
        if special:
            from tokenizers import AddedToken

            tk.add_special_tokens([AddedToken(t, special=True) for t in special])
        return tk, special
    if os.path.exists(p("vocab.txt")):
        from tokenizers import Tokenizer, decoders, models, normalizers, pre_tokenizers, processors

        with open(p("vocab.txt"), encoding="utf-8") as f:
            vocab = {line.rstrip("\n"): i for i, line in enumerate(f)}
        unk = _tok_str(config.get("unk_token")) or "[UNK]"
        tk = Tokenizer(models.WordPiece(vocab, unk_token=unk))
        tk.normalizer = normalizers.BertNormalizer(lowercase=bool(config.get("do_lower_case", True)))
        tk.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
        tk.decoder = decoders.WordPiece()
        cls, sep = _tok_str(config.get("cls_token")) or "[CLS]", _tok_str(config.get("sep_token")) or "[SEP]"
        if cls in vocab and sep in vocab:
            tk.post_processor = processors.TemplateProcessing(single=f"{cls} $A {sep}", pair=f"{cls} $A {sep} $B:1 {sep}:1",
                                                              special_tokens=[(cls, vocab[cls]), (sep, vocab[sep])])
        special = {t: vocab[t] for t in (cls, sep, unk, "[PAD]", "[MASK]") if t in vocab}
        from tokenizers import AddedToken

        tk.add_special_tokens([AddedToken(t, special=True) for t in special])
        config.setdefault("pad_token", "[PAD]")
        return tk, special
    return None


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
        elif (legacy := _legacy_backend(model_dir, config)) is not None:
            tk, special = legacy
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


class SpecialTextView:
    """Text of a generation WITH special tokens, kept next to the plain incremental detokeniser. Until the first special token
    appears both texts are the same string, so nothing is decoded twice; the first special token starts a second incremental
    detokeniser by replaying the ids seen so far (once)."""

    def __init__(self, tokenizer: PreTrainedTokenizer, plain: IncrementalDetokenizer):
        self.tk = tokenizer
        self.plain = plain
        self.own: Optional[IncrementalDetokenizer] = None

    def push(self, token_id: int) -> None:
        """Call BEFORE pushing the same token into the plain detokeniser."""
        if self.own is not None:
            self.own.push(token_id)
        elif self.tk.is_special(token_id):
            self.own = IncrementalDetokenizer(self.tk, skip_special=False)
            for t in self.plain.ids:
                self.own.push(t)
            self.own.push(token_id)

    @property
    def text(self) -> str:
        return self.plain.text if self.own is None else self.own.text

