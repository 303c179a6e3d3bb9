"""Host tier of the prefix cache: snapshots that leave the device banks go to pinned host memory and come back on a hit.

The device banks of the serving backend hold `KVSnapshot`s whose full pages stay in the device page pool.  When a
bank evicts a snapshot, or the scheduler drops one because the pool is short of pages, the snapshot is demoted
here instead of being lost: every full page (the compressed and index rows of all sources for `page_tokens`
positions) is copied into one fixed-size host page, and the small private parts (the partly filled last page, the
window rings, the ratio-2 carry, the logits after the last token) are kept as host tensors.  `csrc/core/hostcache.cc`
owns the host pages: content keys give exact page sharing between snapshots with a common prefix (a page is keyed by a
hash of all tokens up to its end), least recently used snapshots are evicted when the slab pool is full, and store /
restore traffic is budgeted per scheduler tick.  A prompt that extends a demoted snapshot gets fresh device pages
filled from the host pages and continues from the snapshot's end.

Reference: rust/crates/ds41rt-hostcache/src/lib.rs:1-74 (tier, sharing, budgets) and
rust/crates/ds41rt-daemon/src/v41_native_serve/prefix.rs:258-294 (restore shapes).
"""
from __future__ import annotations

import hashlib
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import core as K


class HostSnapshotTier:
    def __init__(self, cache, host_bytes: int, entries: int = 64, store_budget: int = 1 << 62,
                 restore_budget: int = 1 << 62):
        self.cache = cache
        self.sources = sorted(cache.page_rows)
        # one host page = for every source its compressed rows, then its index rows, of one device page
        self.parts = []
        off = 0
        for src in self.sources:
            pr = cache.page_rows[src]
            for pool in (cache.comp[src], cache.idx[src]):
                nbytes = pr * pool[0].numel() * pool.element_size()
                self.parts.append((pool, pr, off, nbytes))
                off += nbytes
        self.page_bytes = max(off, 1)
        self.n_pages = max(1, host_bytes // self.page_bytes)
        self.buf = torch.empty(self.n_pages, self.page_bytes, dtype=torch.uint8)
        if cache.win.device.type == "cuda":
            self.buf = self.buf.pin_memory()
        self.hc = K.HostCache(self.n_pages, self.page_bytes, store_budget, restore_budget)
        self.index = K.PrefixBanks(entries, 1, cache.cfg.window)
        self.meta: Dict[int, dict] = {}
        self.demoted = self.promoted = self.promoted_tokens = 0

    # ------------------------------------------------------------------ helpers
    def _page_keys(self, tokens: Sequence[int], n_pages: int) -> List[int]:
        """Content key of page i: a hash of every token up to the end of the page (its rows depend on all of them)."""
        h = hashlib.blake2b(digest_size=8)
        arr = np.ascontiguousarray(tokens, dtype=np.uint32)
        P = self.cache.page_tokens
        keys = []
        for i in range(n_pages):
            h.update(arr[i * P:(i + 1) * P].tobytes())
            keys.append(int.from_bytes(h.copy().digest(), "little"))
        return keys

    def _copy_page(self, dev_page: int, host_page: int, to_host: bool):
        row = self.buf[host_page]
        for pool, pr, off, nbytes in self.parts:
            dev = pool[dev_page * pr:(dev_page + 1) * pr].view(torch.uint8).view(-1)
            if to_host:
                row[off:off + nbytes].copy_(dev, non_blocking=True)
            else:
                dev.copy_(row[off:off + nbytes], non_blocking=True)

    def _sync(self):
        if self.cache.win.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    def tick(self):
        self.hc.tick()

    # ------------------------------------------------------------------ demote / promote
    def demote(self, tokens: Sequence[int], snap, logits) -> bool:
        """Copy a device snapshot that is about to be dropped.  False: deferred by the budget or no room."""
        tokens = tuple(tokens)
        if not tokens or snap.n_tokens != len(tokens):
            return False
        sid, evicted = self.index.insert(tokens, 0)
        if evicted >= 0:
            self.meta.pop(evicted, None)
            self.hc.drop(evicted)
        if sid < 0:
            return False
        n = len(snap.pages)
        pages: List[int] = []
        if n:
            r, pages, need = self.hc.store(sid, self._page_keys(tokens, n), len(tokens))
            if r <= 0:
                self.index.remove(sid)
                return False
            for dev_page, host_page, copy in zip(snap.pages, pages, need):
                if copy:
                    self._copy_page(dev_page, host_page, to_host=True)
        host = lambda t: None if t is None else t.detach().to("cpu", non_blocking=False)
        self.meta[sid] = {
            "tokens": tokens, "n_pages": n,
            "partial": {src: (host(a), host(b)) for src, (a, b) in snap.partial.items()},
            "rings": host(snap.rings), "pending": {src: host(t) for src, t in snap.pending.items()},
            "logits": host(logits)}
        self._sync()
        self.demoted += 1
        return True

    def lookup(self, prompt: Sequence[int]):
        """Longest demoted snapshot whose tokens are a prefix of `prompt` -> (id, n_tokens, has logits) or None."""
        while True:
            hit = self.index.lookup(prompt)
            if hit is None or not hit["exact"]:
                return None
            sid = hit["id"]
            m = self.meta.get(sid)
            if m is not None and (m["n_pages"] == 0 or self.hc.contains(sid)):
                return sid, len(m["tokens"]), m["logits"] is not None
            self.meta.pop(sid, None)                   # the page pool evicted it behind the index
            self.index.remove(sid)

    def restore_into(self, slot: int, sid: int):
        """Fill an empty `slot` from a demoted snapshot -> (n_tokens, logits on the cache's device or None), or None when
        the device pool is short of pages or the restore budget defers it."""
        m = self.meta.get(sid)
        if m is None:
            return None
        cache = self.cache
        n_tok, n = len(m["tokens"]), m["n_pages"]
        host_pages: List[int] = []
        if n:
            r, host_pages = self.hc.restore(sid, cap=max(n, 1))
            if r <= 0:
                return None
        if not cache.ensure(slot, n_tok if m["partial"] else n * cache.page_tokens):
            return None
        dev_pages = cache.pages_of(slot)
        for dev_page, host_page in zip(dev_pages[:n], host_pages):
            self._copy_page(dev_page, host_page, to_host=False)
        if m["partial"]:
            pg = dev_pages[n]
            for src, (c, ix) in m["partial"].items():
                pr = cache.page_rows[src]
                cache.comp[src][pg * pr: pg * pr + c.shape[0]].copy_(c, non_blocking=True)
                cache.idx[src][pg * pr: pg * pr + ix.shape[0]].copy_(ix, non_blocking=True)
        cache.win[:, slot].copy_(m["rings"], non_blocking=True)
        for src, t in m["pending"].items():
            cache.pending[src][slot].copy_(t, non_blocking=True)
        logits = None if m["logits"] is None else m["logits"].to(cache.win.device, non_blocking=True)
        self._sync()
        self.promoted += 1
        self.promoted_tokens += n_tok
        return n_tok, logits

    def stats(self) -> dict:
        out = self.hc.metrics()
        out.update(page_bytes=self.page_bytes, host_pages=self.n_pages, entries=len(self.meta), demoted=self.demoted,
                   promoted=self.promoted, promoted_tokens=self.promoted_tokens)
        return out
