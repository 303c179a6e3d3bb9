"""Host tier of the prefix cache: snapshots that leave the device banks go to pinned host memory and come back on a hit.

The device banks of the serving backend hold `KVSnapshot`s whose full pages stay in the device page pool.  When a
bank evicts a snapshot, or the scheduler drops one because the pool is short of pages, the snapshot is demoted
here instead of being lost: every full page (the compressed and index rows of all sources for `page_tokens`
positions) is copied into one fixed-size host page, and the small private parts (the partly filled last page, the
window rings, the ratio-2 carry, the logits after the last token) are kept as host tensors.  `csrc/core/hostcache.cc`
owns the host pages: content keys give exact page sharing between snapshots with a common prefix (a page is keyed by a
hash of all tokens up to its end), least recently used snapshots are evicted when the slab pool is full, and store /
restore traffic is budgeted per scheduler tick.  A prompt that extends a demoted snapshot gets fresh device pages
filled from the host pages and continues from the snapshot's end.  A prompt that shares only a leading part with one
gets the rows of that part (whole pages below the cut, the cut page up to the cut) and replays the last window of tokens
before the cut, exactly as a truncated snapshot of the device banks does; only the pages it needs are read and budgeted.

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
        self.part_sources = [src for src in self.sources for _ in range(2)]      # source of every entry of `parts`
        self.page_bytes = max(off, 1)
        self.n_pages = max(1, host_bytes // self.page_bytes)
        self.buf = torch.empty(self.n_pages, self.page_bytes, dtype=torch.uint8)
        if cache.win.device.type == "cuda":
            self.buf = self.buf.pin_memory()
        self.hc = K.HostCache(self.n_pages, self.page_bytes, store_budget, restore_budget)
        self.index = K.PrefixBanks(entries, 1, cache.cfg.window)
        self.meta: Dict[int, dict] = {}
        self.demoted = self.promoted = self.promoted_tokens = self.promoted_partial = 0

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

    def _copy_page(self, dev_page: int, host_page: int, to_host: bool, tokens: Optional[int] = None):
        """One page between the device pools and a host page; `tokens` (host -> device only) stops every source at the
        rows that cover the first `tokens` positions of the page."""
        row = self.buf[host_page]
        P = self.cache.page_tokens
        for (pool, pr, off, nbytes), src in zip(self.parts, self.part_sources):
            rows = pr if tokens is None else (tokens * pr + P - 1) // P
            nb = nbytes // pr * rows
            dev = pool[dev_page * pr: dev_page * pr + rows].view(torch.uint8).view(-1)
            if to_host:
                row[off:off + nb].copy_(dev, non_blocking=True)
            else:
                dev.copy_(row[off:off + nb], non_blocking=True)

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

    def lookup_partial(self, prompt: Sequence[int]):
        """A demoted snapshot that shares only a leading part with `prompt` -> (id, tokens whose rows can be reused) or
        None.  The count is the even boundary below the common part minus one window, which is replayed."""
        hit = self.index.lookup(prompt)
        if hit is None or hit["exact"]:
            return None
        sid = hit["id"]
        m = self.meta.get(sid)
        if m is None or (m["n_pages"] and not self.hc.contains(sid)):
            return None
        n = min(hit["common"], len(prompt) - 1, len(m["tokens"])) // 2 * 2 - self.cache.cfg.window
        return (sid, n) if n > 0 else None

    def restore_prefix_into(self, slot: int, sid: int, n_tokens: int) -> bool:
        """Fill an empty `slot` with the compressed and index rows of the snapshot's first `n_tokens` positions (even,
        below its length).  Rings and carry are not restored: the caller replays from `n_tokens` with a window floor
        there.  False when the device pool is short of pages or the restore budget defers the read."""
        m = self.meta.get(sid)
        cache = self.cache
        if m is None or not (0 < n_tokens <= len(m["tokens"])) or n_tokens % 2:
            return False
        P = cache.page_tokens
        full, rem = divmod(n_tokens, P)
        from_host = min(m["n_pages"], full + (1 if rem else 0))          # the cut page is a host page or the partial part
        host_pages: List[int] = []
        if from_host:
            r, host_pages = self.hc.restore_prefix(sid, from_host)
            if r <= 0:
                return False
        if not cache.ensure(slot, n_tokens):
            return False
        dev_pages = cache.pages_of(slot)
        for i in range(min(full, from_host)):
            self._copy_page(dev_pages[i], host_pages[i], to_host=False)
        if rem:
            if full < m["n_pages"]:
                self._copy_page(dev_pages[full], host_pages[full], to_host=False, tokens=rem)
            else:
                pg = dev_pages[full]
                for src, (c, ix) in m["partial"].items():
                    pr = cache.page_rows[src]
                    rows = (rem * pr + P - 1) // P
                    cache.comp[src][pg * pr: pg * pr + rows].copy_(c[:rows], non_blocking=True)
                    cache.idx[src][pg * pr: pg * pr + rows].copy_(ix[:rows], non_blocking=True)
        self._sync()
        self.promoted_partial += 1
        self.promoted_tokens += n_tokens
        return True

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
                   promoted=self.promoted, promoted_partial=self.promoted_partial, promoted_tokens=self.promoted_tokens)
        return out
