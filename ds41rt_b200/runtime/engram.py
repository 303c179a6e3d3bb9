"""Engram request pipeline: token ids -> compressed ids -> n-gram hashes -> prefetch + gather -> rows for the engine.

One `EngramPipeline` serves an engine: it owns one mmap'd table and one gather thread per Engram layer and one
transactional token history per cache slot.  A pass is three calls:

    ticket = pipe.begin(tokens, slots, is_image)   # hashes (side-effect free), page advice, gather requests
    pipe.apply(ticket, engine)                     # waits for the I/O thread, hands the rows to the engine
    pipe.commit(ticket, accepted_per_slot)         # histories advance by the accepted prefix of each slot's rows

`begin` can be issued as soon as the pass's token ids are known, so the table reads overlap whatever the GPU is still
doing; speculative rows that are rejected leave no trace because only `commit` moves a history.

Reference: rust/crates/ds41rt-loader/src/engram_pipeline.rs:69, engram_tokenizer.rs:87-122 (compressed vocabulary),
rust/crates/ds41rt-core/src/engram.rs:141-283 (history), rust/crates/ds41rt-daemon/src/v41_target_pass.rs:403-442.
"""
from __future__ import annotations

import dataclasses
import re
import unicodedata
from typing import Dict, List, Optional, Sequence

import numpy as np

from .core import EngramHistory
from .engram_io import EngramGather, EngramTable

_WS = re.compile(r"[ \t\r\n]+")


def _normalise(text: str) -> str:
    """NFKC, NFD, accents stripped, lower case, whitespace runs -> one space, outer whitespace stripped; a token that is
    ONLY whitespace stays a single space (so that it does not fall together with the empty token)."""
    t = unicodedata.normalize("NFKC", text)
    t = unicodedata.normalize("NFD", t)
    t = "".join(ch for ch in t if unicodedata.category(ch) != "Mn")
    t = t.lower()
    t = _WS.sub(" ", t)
    if t == " ":
        return " "
    return t.strip()


def compressed_token_ids(token_bytes: Sequence[bytes]) -> np.ndarray:
    """Map every vocabulary id to its Engram id: tokens whose normalised text is equal share one id, ids are handed
    out in vocabulary order.  Tokens that are not valid UTF-8 on their own keep their raw bytes as the key; a token
    whose normalised text is empty keeps its original text."""
    keys: Dict[object, int] = {}
    out = np.zeros(len(token_bytes), dtype=np.uint32)
    for i, raw in enumerate(token_bytes):
        try:
            text = raw.decode("utf-8")
            norm = _normalise(text)
            key: object = norm if norm != "" else text
        except UnicodeDecodeError:
            key = raw
        out[i] = keys.setdefault(key, len(keys))
    return out


@dataclasses.dataclass
class _Pass:
    tokens: List[int]                 # compressed ids, -1 = image row
    slots: List[int]
    tickets: List[Optional[int]]      # one gather ticket per layer (None: filled synchronously)
    ids: List[np.ndarray]             # per layer, [rows * rows_per_token] table row ids
    text_mask: np.ndarray


class EngramPipeline:
    def __init__(self, layers: Sequence[int], tables: Sequence[EngramTable], token_map: Optional[np.ndarray] = None,
                 pad_id: int = 2, max_rows: int = 64, gather_slots: int = 4, fold: bool = False,
                 timeout: float = 30.0):
        """`layers[i]` is the decoder layer served by `tables[i]` (hash family i).  `token_map` maps vocabulary ids to
        compressed ids (identity when None).  `fold` reduces row ids modulo the table size, for tables smaller than
        the hash range (random-init models and tests)."""
        assert len(layers) == len(tables) and 1 <= len(layers) <= 2
        self.layers, self.tables, self.map = list(layers), list(tables), token_map
        self.pad, self.fold, self.timeout, self.max_rows = pad_id, fold, timeout, max_rows
        self.gathers = [EngramGather(t, slots=gather_slots, max_rows=24 * max_rows) for t in tables]
        self.hist: Dict[int, EngramHistory] = {}
        self.passes = 0

    # ---------------------------------------------------------------- histories
    def history(self, slot: int) -> EngramHistory:
        if slot not in self.hist:
            self.hist[slot] = EngramHistory(self.pad)
        return self.hist[slot]

    def release(self, slot: int) -> None:
        self.hist.pop(slot, None)

    def fork(self, slot: int) -> EngramHistory:
        """A copy of a slot's history (kept with a KV snapshot)."""
        return self.history(slot).fork()

    def adopt(self, slot: int, hist: EngramHistory) -> None:
        """Continue `slot` from a stored history (the counterpart of a KV snapshot restore)."""
        self.hist[slot] = hist.fork()

    def reset(self, slot: int, tokens: Sequence[int], is_image: Optional[Sequence[bool]] = None) -> None:
        """Start `slot` from a history that has seen `tokens` (`is_image` marks image rows among them): used when a
        request continues from a stored KV snapshot of those tokens."""
        h = EngramHistory(self.pad)
        comp = [self.compress(t, bool(is_image[i]) if is_image is not None else False) for i, t in enumerate(tokens)]
        h.commit(comp, len(comp))
        self.hist[slot] = h

    # ---------------------------------------------------------------- one pass
    def compress(self, token: int, is_image: bool = False) -> int:
        if is_image:
            return -1
        return int(self.map[token]) if self.map is not None else int(token)

    def begin(self, tokens: Sequence[int], slots: Sequence[int], is_image: Optional[Sequence[bool]] = None) -> _Pass:
        """Rows of one pass in pass order; rows of the same slot must be consecutive positions of that request."""
        n = len(tokens)
        assert n == len(slots) and n <= self.max_rows
        img = list(is_image) if is_image is not None else [False] * n
        comp = [self.compress(t, im) for t, im in zip(tokens, img)]
        hashes = np.zeros((n, 2, 24), dtype=np.uint64)
        by_slot: Dict[int, List[int]] = {}
        for i, s in enumerate(slots):
            by_slot.setdefault(s, []).append(i)
        for s, rows in by_slot.items():
            hashes[rows] = self.history(s).prepare([comp[i] for i in rows])
        ids, tickets = [], []
        for li, (table, gather) in enumerate(zip(self.tables, self.gathers)):
            a = hashes[:, li, :].reshape(-1)
            if self.fold:
                a = a % np.uint64(table.rows)
            a = np.ascontiguousarray(a)
            table.prefetch(a)
            ids.append(a)
            tickets.append(gather.submit(a))
        self.passes += 1
        return _Pass(comp, list(slots), tickets, ids, np.array([0 if im else 1 for im in img], dtype=np.uint8))

    def rows(self, p: _Pass, li: int) -> np.ndarray:
        """Gathered rows of layer index `li` for pass `p`: uint8 [rows * 24, row_bytes] (valid until finish())."""
        gather = self.gathers[li]
        if p.tickets[li] is None:                       # the pool was full at begin(): retry now, then wait
            p.tickets[li] = gather.submit(p.ids[li])
            if p.tickets[li] is None:
                raise RuntimeError("engram gather pool exhausted")
        return gather.wait(p.tickets[li], self.timeout)

    def apply(self, p: _Pass, engine) -> None:
        for li, layer in enumerate(self.layers):
            if layer in engine.engram:
                engine.set_engram_rows(layer, self.rows(p, li), p.text_mask)
        self.finish(p)

    def finish(self, p: _Pass) -> None:
        for li, gather in enumerate(self.gathers):
            if p.tickets[li] is not None:
                gather.release(p.tickets[li])
                p.tickets[li] = None

    def cancel(self, p: _Pass) -> None:
        for li, gather in enumerate(self.gathers):
            if p.tickets[li] is not None:
                gather.cancel(p.tickets[li])
                gather.release(p.tickets[li])
                p.tickets[li] = None

    def commit(self, p: _Pass, accepted: Optional[Dict[int, int]] = None) -> None:
        """Advance each slot's history by the first `accepted[slot]` of its rows in the pass (all of them when the
        slot is not named)."""
        by_slot: Dict[int, List[int]] = {}
        for i, s in enumerate(p.slots):
            by_slot.setdefault(s, []).append(i)
        for s, rows in by_slot.items():
            toks = [p.tokens[i] for i in rows]
            k = len(toks) if accepted is None or s not in accepted else int(accepted[s])
            self.history(s).commit(toks, k)

    def stats(self) -> dict:
        return {"passes": self.passes, "gather": [g.stats() for g in self.gathers]}

    def close(self) -> None:
        for g in self.gathers:
            g.close()
        for t in self.tables:
            t.close()
