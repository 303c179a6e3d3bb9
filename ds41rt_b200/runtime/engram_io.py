"""Engram tables on the host: mmap'd rows, prefetch advice and the gather thread (csrc/core/engram_io.cc).

Also a row-delivery benchmark for sizing the pipeline against a storage device:

    python -m ds41rt_b200.runtime.engram_io TABLE.bin --rows N [--row-bytes 264] [--tokens 64] [--mode willneed]
                                            [--cache cold|warm] [--iters 20] [--threads 8]

times the delivery of the records that passes of `tokens` rows need (24 hashed ids per token, sorted and de-duplicated)
through the mapping (`mmap`), with page advice first (`willneed`), with one pread per record (`pread`) or with preads
over threads (`pread-mt`).  `--cache cold` drops this file's pages from the page cache before every pass
(`EngramTable.evict`, file-scoped advice; no system-wide cache drop) and reports the resident fraction it achieved.
Counterpart of the reference's scripts/native/bench-engram-io.cpp and scripts/native/drop-page-cache.c.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Optional, Sequence

import numpy as np

from ..ops import lib


def _core():
    c = lib.core()
    if not getattr(c, "_engram_io_ready", False):
        c.ds41_engram_table_open.restype = C.c_void_p
        c.ds41_engram_table_open.argtypes = [C.c_char_p, C.c_uint64, C.c_uint32, C.POINTER(C.c_int)]
        c.ds41_engram_table_close.argtypes = [C.c_void_p]
        c.ds41_engram_prefetch.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        c.ds41_engram_table_evict.argtypes = [C.c_void_p]
        c.ds41_engram_table_resident.restype = C.c_double
        c.ds41_engram_table_resident.argtypes = [C.c_void_p]
        c.ds41_engram_io_bench.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64,
                                           C.c_void_p]
        c.ds41_engram_gather_create.restype = C.c_void_p
        c.ds41_engram_gather_create.argtypes = [C.c_void_p, C.c_int, C.c_int]
        c.ds41_engram_gather_destroy.argtypes = [C.c_void_p]
        c.ds41_engram_gather_submit.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        c.ds41_engram_gather_poll.argtypes = [C.c_void_p, C.c_int]
        c.ds41_engram_gather_data.restype = C.c_void_p
        c.ds41_engram_gather_data.argtypes = [C.c_void_p, C.c_int]
        c.ds41_engram_gather_cancel.argtypes = [C.c_void_p, C.c_int]
        c.ds41_engram_gather_release.argtypes = [C.c_void_p, C.c_int]
        c.ds41_engram_gather_stats.argtypes = [C.c_void_p, C.c_void_p]
        c._engram_io_ready = True
    return c


class EngramTable:
    """A flat file of `rows` records of `row_bytes` bytes, mapped read-only; the size must match exactly."""

    def __init__(self, path: str, rows: int, row_bytes: int = 264):
        err = C.c_int(0)
        self.h = _core().ds41_engram_table_open(path.encode(), rows, row_bytes, C.byref(err))
        if not self.h:
            raise OSError({1: "bad arguments", 2: "cannot open", 3: "file size does not match rows x row_bytes",
                           4: "mmap failed"}.get(err.value, str(err.value)) + f": {path}")
        self.rows, self.row_bytes = rows, row_bytes

    def prefetch(self, ids: Sequence[int]) -> int:
        a = np.ascontiguousarray(ids, dtype=np.uint64)
        r = _core().ds41_engram_prefetch(self.h, a.ctypes.data, a.size)
        if r < 0:
            raise IndexError("engram row id out of range")
        return r

    def evict(self) -> None:
        """Drop this file's pages from the page cache (advice scoped to the file; the next reads come from storage)."""
        rc = _core().ds41_engram_table_evict(self.h)
        if rc != 0:
            raise OSError(f"page-cache advice failed ({rc})")

    def resident(self) -> float:
        """Fraction of the table's pages that are in memory."""
        return float(_core().ds41_engram_table_resident(self.h))

    MODES = {"mmap": 0, "willneed": 1, "pread": 2, "pread-mt": 3}

    def bench(self, tokens: int = 64, rows_per_token: int = 24, mode: str = "willneed", threads: int = 8,
              iters: int = 20, cold: bool = False, seed: int = 0) -> dict:
        """Time `iters` synthetic passes of `tokens` rows -> {"mean_us", "min_us", "max_us", "records_per_pass", ...}."""
        out = (C.c_double * 5)()
        rc = _core().ds41_engram_io_bench(self.h, tokens, rows_per_token, self.MODES[mode], threads, iters, int(cold),
                                          seed, out)
        if rc != 0:
            raise OSError({-1: "bad arguments", -2: "read error"}.get(rc, str(rc)))
        recs = out[3]
        return {"mode": mode, "cache": "cold" if cold else "warm", "tokens": tokens, "records_per_pass": round(recs, 1),
                "mean_us": round(out[0], 1), "min_us": round(out[1], 1), "max_us": round(out[2], 1),
                "us_per_record": round(out[0] / max(recs, 1.0), 3),
                "mb_per_s": round(recs * self.row_bytes / max(out[0], 1e-9), 1), "iters": iters,
                "threads": threads if mode == "pread-mt" else 1}

    def close(self):
        if self.h:
            _core().ds41_engram_table_close(self.h)
            self.h = None


class EngramGather:
    """Bounded pool of staging slots filled by one I/O thread.  submit() -> ticket or None (pool exhausted)."""

    def __init__(self, table: EngramTable, slots: int = 4, max_rows: int = 24 * 64):
        self.table, self.max_rows = table, max_rows
        self.h = _core().ds41_engram_gather_create(table.h, slots, max_rows)
        if not self.h:
            raise MemoryError("cannot create the engram gather pool")
        self._n = {}

    def submit(self, ids: Sequence[int]) -> Optional[int]:
        a = np.ascontiguousarray(ids, dtype=np.uint64)
        t = _core().ds41_engram_gather_submit(self.h, a.ctypes.data, a.size)
        if t == -2:
            raise IndexError("engram row id out of range or request larger than a slot")
        if t < 0:
            return None
        self._n[t] = a.size
        return t

    def poll(self, ticket: int) -> Optional[bool]:
        """True ready, False pending, None cancelled."""
        r = _core().ds41_engram_gather_poll(self.h, ticket)
        if r == -2:
            raise KeyError(ticket)
        return None if r == -1 else bool(r)

    def wait(self, ticket: int, timeout: float = 30.0) -> np.ndarray:
        """Rows of the request as a uint8 view [n, row_bytes] of the staging slot (valid until release)."""
        end = time.time() + timeout
        while True:
            st = self.poll(ticket)
            if st:
                break
            if st is None:
                raise RuntimeError("engram gather was cancelled")
            if time.time() > end:
                raise TimeoutError("engram gather did not finish")
            time.sleep(0.0002)
        ptr = _core().ds41_engram_gather_data(self.h, ticket)
        n = self._n[ticket]
        buf = (C.c_uint8 * (n * self.table.row_bytes)).from_address(ptr)
        return np.frombuffer(buf, dtype=np.uint8).reshape(n, self.table.row_bytes)

    def cancel(self, ticket: int):
        _core().ds41_engram_gather_cancel(self.h, ticket)

    def release(self, ticket: int) -> bool:
        ok = _core().ds41_engram_gather_release(self.h, ticket) == 0
        if ok:
            self._n.pop(ticket, None)
        return ok

    def stats(self) -> dict:
        out = (C.c_uint64 * 4)()
        _core().ds41_engram_gather_stats(self.h, out)
        return {"requests": out[0], "rows_copied": out[1], "refused": out[2], "cancelled": out[3]}

    def close(self):
        if self.h:
            _core().ds41_engram_gather_destroy(self.h)
            self.h = None


def main(argv=None) -> int:
    import argparse
    import json
    ap = argparse.ArgumentParser(description="Engram row-delivery benchmark (host only)")
    ap.add_argument("table")
    ap.add_argument("--rows", type=int, required=True)
    ap.add_argument("--row-bytes", type=int, default=264)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--rows-per-token", type=int, default=24)
    ap.add_argument("--mode", default="willneed", choices=sorted(EngramTable.MODES))
    ap.add_argument("--cache", default="warm", choices=["cold", "warm"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--threads", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    t = EngramTable(args.table, args.rows, args.row_bytes)
    try:
        if args.cache == "warm":
            t.bench(args.tokens, args.rows_per_token, "mmap", 1, 2, False, args.seed)       # touch once
        else:
            t.evict()
        before = t.resident()
        out = t.bench(args.tokens, args.rows_per_token, args.mode, args.threads, args.iters, args.cache == "cold",
                      args.seed)
        out["resident_before"] = round(before, 4)
        out["resident_after"] = round(t.resident(), 4)
        print(json.dumps(out))
    finally:
        t.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
