"""Request-level glue for guided decoding: picks the guide for a request and caches vocabularies / indexes per model.

One mode per request (choice | regex | json), json goes through the schema->regex builder, regex uses the lazy index by
default; the vocabulary is built once per model by decoding every token id except the EOS ids, and indexes are cached by
pattern (reference: core/.../guided/LogitsProcessorFactory.java:31-33,42-69,84-138, GuideLogitsProcessor.java:23-47).
"""
from __future__ import annotations

import json
import threading
from typing import Optional

from ..params import GeneratorParameters
from .index import DEFAULT_SETTINGS, ChoiceGuide, Guide, Index, IndexGuide, LazyIndex, SketchesSettings, Vocabulary
from .json_schema import schema_to_regex


class LogitsProcessorFactory:
    def __init__(self, tokenizer, eos_ids, vocab_size: int, settings: SketchesSettings = DEFAULT_SETTINGS, max_cached: int = 64):
        self.tokenizer = tokenizer
        self.eos_ids = tuple(sorted(set(int(e) for e in eos_ids)))
        self.vocab_size = vocab_size
        self.settings = settings
        self._vocab: Optional[Vocabulary] = None
        self._indexes: dict[str, LazyIndex] = {}
        self._json_regex: dict[str, str] = {}
        self._lock = threading.Lock()
        self.max_cached = max_cached
        self.metrics = {"index_hits": 0, "index_builds": 0}

    def vocabulary(self) -> Vocabulary:
        with self._lock:
            if self._vocab is None:
                self._vocab = Vocabulary.from_tokenizer(self.tokenizer, self.eos_ids, self.vocab_size)
            return self._vocab

    def index_for(self, pattern: str) -> LazyIndex:
        vocab = self.vocabulary()
        with self._lock:
            idx = self._indexes.get(pattern)
            if idx is not None:
                self.metrics["index_hits"] += 1
                return idx
        idx = (Index if self.settings.mode == "EAGER" else LazyIndex)(pattern, vocab, self.settings)
        with self._lock:
            if len(self._indexes) >= self.max_cached:
                self._indexes.pop(next(iter(self._indexes)))
            self._indexes[pattern] = idx
            self.metrics["index_builds"] += 1
        return idx

    def create(self, params: GeneratorParameters) -> Optional[Guide]:
        modes = [m for m in (params.guided_choice, params.guided_regex, params.guided_json) if m is not None]
        if not modes:
            return None
        if len(modes) > 1:
            raise ValueError("only one guided decoding mode may be set per request")
        if params.guided_choice is not None:
            enc = [self.tokenizer.encode(c) for c in params.guided_choice]
            return ChoiceGuide(enc, self.eos_ids, self.vocab_size)
        if params.guided_json is not None:
            key = params.guided_json if isinstance(params.guided_json, str) else json.dumps(params.guided_json, sort_keys=False)
            pattern = self._json_regex.get(key)
            if pattern is None:
                pattern = schema_to_regex(params.guided_json)
                self._json_regex[key] = pattern
        else:
            pattern = params.guided_regex
        return IndexGuide(self.index_for(pattern))
