"""Guided decoding automata: regex -> DFA, token vocabulary trie, lazy / eager per-state token index, guides.

Semantics follow the reference's ``sketches-core`` (sketches-core/src/main/java/io/teknek/sketches/guide/LazyIndex.java:20-172,
Index.java:36-131, ChoiceGuide.java:20-49, SketchesSettings.java:16-17): the regex must match the WHOLE output; a token is
allowed in DFA state ``s`` iff walking all of its characters from ``s`` stays inside the automaton, and the landing state is
the next state; accepting states additionally allow every EOS id (as a self-loop); empty-text tokens are never allowed;
per-state transitions are computed on demand and memoised (lazy) or up-front with state / transition limits (eager).
The regex dialect is that of ``interegular`` (Python ``re`` subset without look-around / back-references) instead of
dk.brics.automaton. Masks are int32 allow-bitmasks ``[ceil(V/32)]`` that the sampler kernels consume directly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional

import torch


@dataclass(frozen=True)
class SketchesSettings:
    max_regex_length: int = 10_000
    max_index_states: int = 10_000
    max_index_transitions: int = 2_000_000
    mode: str = "LAZY"  # LAZY | EAGER


DEFAULT_SETTINGS = SketchesSettings()


class Vocabulary:
    """token id -> decoded text (EOS ids excluded), plus a character trie over the token texts."""

    def __init__(self, tokens: dict[int, str], eos_ids: Iterable[int], vocab_size: Optional[int] = None):
        self.eos_ids = tuple(sorted(set(int(e) for e in eos_ids)))
        self.tokens = {int(i): s for i, s in tokens.items() if int(i) not in self.eos_ids and s}
        self.vocab_size = vocab_size or (max(list(self.tokens) + list(self.eos_ids)) + 1 if (self.tokens or self.eos_ids) else 0)
        # trie: node = [children dict char -> node index, token ids ending here]
        self.children: list[dict] = [{}]
        self.ends: list[list[int]] = [[]]
        for tid, s in self.tokens.items():
            n = 0
            for ch in s:
                nxt = self.children[n].get(ch)
                if nxt is None:
                    nxt = len(self.children)
                    self.children[n][ch] = nxt
                    self.children.append({})
                    self.ends.append([])
                n = nxt
            self.ends[n].append(tid)

    @staticmethod
    def from_tokenizer(tokenizer, eos_ids: Iterable[int], vocab_size: Optional[int] = None) -> "Vocabulary":
        V = vocab_size or tokenizer.vocab_size
        eos = set(int(e) for e in eos_ids)
        toks = {}
        for i in range(min(V, tokenizer.vocab_size)):
            if i in eos:
                continue
            s = tokenizer.decode([i])
            if s and "�" not in s:
                toks[i] = s
        return Vocabulary(toks, eos, V)

    @property
    def words(self) -> int:
        return (self.vocab_size + 31) // 32


def _set_bits(ids: Iterable[int], words: int) -> torch.Tensor:
    m = torch.zeros(words, dtype=torch.int64)
    idx = torch.tensor(sorted(set(int(i) for i in ids)), dtype=torch.int64)
    if idx.numel():
        # OR the bits of each word together: group by word
        w = idx >> 5
        b = torch.ones_like(idx) << (idx & 31)
        order = torch.argsort(w)
        w, b = w[order], b[order]
        uw, inv = torch.unique_consecutive(w, return_inverse=True)
        acc = torch.zeros(uw.numel(), dtype=torch.int64)
        # OR == sum here because every (word, bit) pair is distinct
        acc.index_add_(0, inv, b)
        m[uw] = acc
    m = torch.where(m >= 2**31, m - 2**32, m)
    return m.to(torch.int32)


class RegexDFA:
    def __init__(self, pattern: str, settings: SketchesSettings = DEFAULT_SETTINGS):
        import interegular
        from interegular.fsm import anything_else

        if len(pattern) > settings.max_regex_length:
            raise ValueError(f"regex longer than {settings.max_regex_length} characters")
        try:
            fsm = interegular.parse_pattern(pattern).to_fsm().reduce()
        except Exception as e:  # noqa: BLE001 - the parser's own exception types carry no message
            raise ValueError(f"cannot compile guided regex {pattern[:80]!r}: {type(e).__name__} {e}".rstrip()) from e
        self.initial = fsm.initial
        self.finals = frozenset(fsm.finals)
        self.map = fsm.map
        self.alphabet = fsm.alphabet
        self._else = fsm.alphabet[anything_else] if anything_else in fsm.alphabet else None
        self.num_states = len(fsm.states)

    def step(self, state: int, ch: str) -> Optional[int]:
        sym = self.alphabet._symbol_mapping.get(ch, self._else)
        if sym is None:
            return None
        return self.map.get(state, {}).get(sym)

    def live_states(self) -> set:
        """States from which an accepting state is reachable."""
        rev: dict[int, set] = {}
        for s, tr in self.map.items():
            for _, t in tr.items():
                rev.setdefault(t, set()).add(s)
        live, stack = set(self.finals), list(self.finals)
        while stack:
            t = stack.pop()
            for s in rev.get(t, ()):
                if s not in live:
                    live.add(s)
                    stack.append(s)
        return live


class LazyIndex:
    """Per-state ``{token id -> next state}`` computed on demand by walking the vocabulary trie through the DFA."""

    def __init__(self, pattern: str, vocab: Vocabulary, settings: SketchesSettings = DEFAULT_SETTINGS):
        self.dfa = RegexDFA(pattern, settings)
        self.vocab = vocab
        self.settings = settings
        self._live = self.dfa.live_states()
        self._trans: dict[int, dict[int, int]] = {}
        self._masks: dict[int, torch.Tensor] = {}
        self.transitions_computed = 0

    @property
    def initial(self) -> int:
        return self.dfa.initial

    def is_final(self, state: int) -> bool:
        return state in self.dfa.finals

    def transitions(self, state: int) -> dict[int, int]:
        t = self._trans.get(state)
        if t is not None:
            return t
        out: dict[int, int] = {}
        ch, ends = self.vocab.children, self.vocab.ends
        stack = [(0, state)]
        while stack:
            node, st = stack.pop()
            for c, nxt in ch[node].items():
                s2 = self.dfa.step(st, c)
                if s2 is None or s2 not in self._live:
                    continue
                for tid in ends[nxt]:
                    out[tid] = s2
                if ch[nxt]:
                    stack.append((nxt, s2))
        if self.is_final(state):
            for e in self.vocab.eos_ids:
                out[e] = state
        self._trans[state] = out
        self.transitions_computed += len(out)
        return out

    def mask(self, state: int) -> torch.Tensor:
        m = self._masks.get(state)
        if m is None:
            m = _set_bits(self.transitions(state).keys(), self.vocab.words)
            self._masks[state] = m
        return m

    def mask_on(self, state: int, device) -> torch.Tensor:
        """The allow-bitmask of ``state`` as a tensor on ``device`` (uploaded once per state and kept)."""
        cache = self.__dict__.setdefault("_dev_masks", {})
        key = (state, str(device))
        m = cache.get(key)
        if m is None:
            m = self.mask(state).to(device)
            cache[key] = m
        return m

    def next_state(self, state: int, token: int) -> Optional[int]:
        return self.transitions(state).get(token)


class Index(LazyIndex):
    """Eager index: every reachable state is expanded at construction, within the state / transition limits."""

    def __init__(self, pattern: str, vocab: Vocabulary, settings: SketchesSettings = DEFAULT_SETTINGS):
        super().__init__(pattern, vocab, settings)
        seen, todo = {self.initial}, [self.initial]
        total = 0
        while todo:
            s = todo.pop()
            tr = self.transitions(s)
            total += len(tr)
            if len(seen) > settings.max_index_states:
                raise ValueError(f"index exceeds {settings.max_index_states} states")
            if total > settings.max_index_transitions:
                raise ValueError(f"index exceeds {settings.max_index_transitions} transitions")
            for t in set(tr.values()):
                if t not in seen:
                    seen.add(t)
                    todo.append(t)
        self.states = seen


class Guide:
    def allowed_mask(self) -> torch.Tensor:
        raise NotImplementedError

    def accept(self, token: int) -> None:
        raise NotImplementedError

    def is_complete(self) -> bool:
        return False

    def allowed_tokens(self) -> list[int]:
        m = self.allowed_mask().to(torch.int64) & 0xFFFFFFFF
        out = []
        for w, v in enumerate(m.tolist()):
            while v:
                b = (v & -v).bit_length() - 1
                out.append(w * 32 + b)
                v &= v - 1
        return out


class IndexGuide(Guide):
    """Walks a (lazy or eager) index. ``is_complete`` stays False: regex / JSON guides end through EOS."""

    def __init__(self, index: LazyIndex):
        self.index = index
        self.state = index.initial
        self.finished = False

    def allowed_mask(self) -> torch.Tensor:
        return self.index.mask(self.state)

    def allowed_mask_on(self, device) -> torch.Tensor:
        return self.index.mask_on(self.state, device)

    def accept(self, token: int) -> None:
        if token in self.index.vocab.eos_ids:
            self.finished = True
            return
        nxt = self.index.next_state(self.state, token)
        if nxt is None:
            raise ValueError(f"token {token} is not allowed in guide state {self.state}")
        self.state = nxt


class ChoiceGuide(Guide):
    """Prefix match over the token-id encodings of each choice; EOS is allowed once a choice is complete."""

    def __init__(self, choices: list[list[int]], eos_ids: Iterable[int], vocab_size: int):
        if not choices:
            raise ValueError("guided_choice needs at least one choice")
        self.choices = [list(c) for c in choices]
        self.eos_ids = tuple(eos_ids)
        self.words = (vocab_size + 31) // 32
        self.taken: list[int] = []
        self.done = False

    def _candidates(self) -> list[list[int]]:
        n = len(self.taken)
        return [c for c in self.choices if c[:n] == self.taken]

    def allowed_mask(self) -> torch.Tensor:
        n = len(self.taken)
        allowed = set()
        for c in self._candidates():
            if len(c) > n:
                allowed.add(c[n])
            else:
                allowed.update(self.eos_ids)
        return _set_bits(allowed, self.words)

    def accept(self, token: int) -> None:
        if token in self.eos_ids:
            self.done = True
            return
        self.taken.append(token)
        if not self._candidates():
            raise ValueError(f"token {token} does not continue any choice")

    def is_complete(self) -> bool:
        n = len(self.taken)
        cands = self._candidates()
        return self.done or (len(cands) >= 1 and all(len(c) == n for c in cands))
