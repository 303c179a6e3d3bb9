"""Constrained decoding: grammar compilation, matchers and per-step token masks (bindings of csrc/core/grammar.cc)
plus the request-level constraint objects the serving engine uses.

`TokenConstraint` mirrors the behaviour of the reference's serving constraints
(rust/crates/ds41rt-api/src/native_v41/constraints.rs:8-68): an optional "thinking" prefix (any tokens until the
end-of-thinking token), then the content grammar; per-round verification masks come from forks of the authoritative
matcher, and a proposal is truncated to its grammar-accepted prefix.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..ops import lib as _lib

_c = None


def _core():
    global _c
    if _c is None:
        c = _lib.core()
        for name in ("ds41_vocab_new", "ds41_grammar_compile", "ds41_matcher_new", "ds41_matcher_fork"):
            getattr(c, name).restype = C.c_void_p
        _c = c
    return _c


class GrammarError(ValueError):
    pass


class Vocab:
    """Byte strings of every token id (empty for special tokens, which a grammar never allows by content)."""

    def __init__(self, token_bytes: Sequence[bytes]):
        self.size = len(token_bytes)
        data = b"".join(token_bytes)
        offs = np.zeros(self.size + 1, dtype=np.int64)
        np.cumsum([len(b) for b in token_bytes], out=offs[1:])
        buf = np.frombuffer(data, dtype=np.uint8) if data else np.zeros(1, dtype=np.uint8)
        self.h = C.c_void_p(_core().ds41_vocab_new(buf.ctypes.data_as(C.c_void_p), offs.ctypes.data_as(C.c_void_p),
                                                   self.size))
        self.token_bytes = list(token_bytes)
        self.words = (self.size + 31) // 32

    def __del__(self):
        try:
            _core().ds41_vocab_free(self.h)
        except Exception:
            pass


class Grammar:
    def __init__(self, description):
        text = description if isinstance(description, str) else json.dumps(description)
        err = C.create_string_buffer(512)
        h = _core().ds41_grammar_compile(text.encode(), err, 512)
        if not h:
            raise GrammarError(err.value.decode() or "grammar compilation failed")
        self.h = C.c_void_p(h)

    def __del__(self):
        try:
            _core().ds41_grammar_free(self.h)
        except Exception:
            pass

    @staticmethod
    def json_schema(schema: dict) -> "Grammar":
        return Grammar({"schema": schema})

    @staticmethod
    def regex(pattern: str) -> "Grammar":
        return Grammar({"regex": pattern})

    @staticmethod
    def json_object() -> "Grammar":
        return Grammar({"schema": {"type": "object"}})


class Matcher:
    def __init__(self, grammar: Grammar, _handle=None):
        self.grammar = grammar
        self.h = C.c_void_p(_handle if _handle is not None else _core().ds41_matcher_new(grammar.h))

    def __del__(self):
        try:
            _core().ds41_matcher_free(self.h)
        except Exception:
            pass

    def fork(self) -> "Matcher":
        return Matcher(self.grammar, _core().ds41_matcher_fork(self.h))

    def reset(self):
        _core().ds41_matcher_reset(self.h)

    def accept_bytes(self, data: bytes) -> bool:
        return bool(_core().ds41_matcher_accept_bytes(self.h, data, len(data)))

    def accept_token(self, vocab: Vocab, token: int) -> bool:
        return bool(_core().ds41_matcher_accept_token(self.h, vocab.h, token))

    @property
    def can_finish(self) -> bool:
        return bool(_core().ds41_matcher_can_finish(self.h))

    @property
    def terminated(self) -> bool:
        return bool(_core().ds41_matcher_is_terminated(self.h))

    @property
    def threads(self) -> int:
        return int(_core().ds41_matcher_threads(self.h))

    def fill_mask(self, vocab: Vocab, stop_token: int = -1, out: Optional[np.ndarray] = None) -> np.ndarray:
        if out is None:
            out = np.zeros(vocab.words, dtype=np.uint32)
        _core().ds41_matcher_fill_mask(self.h, vocab.h, out.ctypes.data_as(C.c_void_p), stop_token)
        return out


def mask_allows(mask: np.ndarray, token: int) -> bool:
    return bool((int(mask[token >> 5]) >> (token & 31)) & 1)


class TokenConstraint:
    """Request-level constraint: [thinking prefix] + content grammar, evaluated on token ids."""

    def __init__(self, vocab: Vocab, grammar: Optional[Grammar], eos: int, think_end: Optional[int] = None,
                 thinking: bool = False):
        self.vocab, self.grammar, self.eos, self.think_end = vocab, grammar, eos, think_end
        self.in_thinking = thinking and think_end is not None
        self.matcher = Matcher(grammar) if grammar is not None else None
        self.finished = False

    def fork(self) -> "TokenConstraint":
        c = TokenConstraint.__new__(TokenConstraint)
        c.vocab, c.grammar, c.eos, c.think_end = self.vocab, self.grammar, self.eos, self.think_end
        c.in_thinking, c.finished = self.in_thinking, self.finished
        c.matcher = self.matcher.fork() if self.matcher is not None else None
        return c

    def mask(self) -> Optional[np.ndarray]:
        """Allow-mask for the next token, or None when anything is allowed."""
        if self.in_thinking:
            m = np.full(self.vocab.words, 0xFFFFFFFF, dtype=np.uint32)
            m[self.eos >> 5] &= ~np.uint32(1 << (self.eos & 31))     # thinking must be closed explicitly
            return m
        if self.matcher is None:
            return None
        return self.matcher.fill_mask(self.vocab, stop_token=self.eos)

    def accept(self, token: int) -> bool:
        if self.in_thinking:
            if token == self.think_end:
                self.in_thinking = False
            return token != self.eos
        if token == self.eos:
            ok = self.matcher is None or self.matcher.can_finish
            self.finished = self.finished or ok
            return ok
        if self.matcher is None:
            return True
        return self.matcher.accept_token(self.vocab, token)

    def truncate_proposal(self, drafts: Sequence[int]) -> List[int]:
        """Longest prefix of `drafts` the grammar accepts (the authoritative matcher is not mutated).
        A draft that completes the grammar does NOT end the proposal: only a rejected token does."""
        probe = self.fork()
        keep = []
        for t in drafts:
            if not probe.accept(t):
                break
            keep.append(t)
        return keep

    def row_masks(self, inputs: Sequence[int]) -> List[Optional[np.ndarray]]:
        """Masks for a verification chunk: row i's mask applies after consuming inputs[1..i] (inputs[0] is the
        anchor, which the authoritative matcher has already accepted)."""
        probe = self.fork()
        out = [probe.mask()]
        for t in inputs[1:]:
            if not probe.accept(t):
                break
            out.append(probe.mask())
        return out


def byte_level_vocab(tokens: Dict[str, int], size: int, specials: Sequence[int] = ()) -> Vocab:
    """Vocabulary table from a byte-level BPE token->id map (GPT-2 style printable-byte alphabet)."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    dec = {chr(c): b for b, c in zip(bs, cs)}
    table = [b""] * size
    skip = set(specials)
    for tok, i in tokens.items():
        if i in skip or i >= size:
            continue
        try:
            table[i] = bytes(dec[ch] for ch in tok)
        except KeyError:
            table[i] = tok.encode("utf-8")
    return Vocab(table)
