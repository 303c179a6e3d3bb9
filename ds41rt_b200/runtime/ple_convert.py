"""Convert an Engram table from FP8 records to NVFP4 records on the CPU, streamed and resumable.

    python -m ds41rt_b200.runtime.ple_convert SRC.bin DST.bin --rows N [--dim 256] [--threads 8] [--chunk-rows 262144]

Source record: `dim` E4M3 bytes + `dim / 32` UE8M0 scale bytes (264 bytes for dim 256, the layout that
`loader.official.export_engram_table` writes).  Output record: `dim / 2` bytes of E2M1 pairs (even element in the low
nibble) + `dim / 16` E4M3 scale bytes (144 bytes for dim 256); the one fp32 scale of the table goes to `DST.bin.json`
together with the geometry, and `serve --engram-format nvfp4` reads it from there.

Two passes over the source in chunks of `chunk_rows` records, both through memory maps, so the resident set stays at a
chunk whatever the table size: pass 1 finds the table's largest magnitude (-> scale = amax / (6 * 448)), pass 2
quantises (native code in csrc/core/ple_convert.cc, `threads` host threads).  After every chunk the progress file
`DST.bin.progress.json` is rewritten atomically; a later run with the same source (size, mtime and a hash of its first and
last MiB) and the same geometry picks up after the last finished chunk.  No GPU is used.
Counterpart of the reference's CPU-only table conversion (quantization/fp4ple.py + quantization/ple_nvfp4_cpu.cpp).
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import json
import math
import os
import time

import numpy as np


def _core():
    from ..ops import lib
    core = lib.core()
    core.ds41_ple_scan.restype = C.c_int
    core.ds41_ple_scan.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float)]
    core.ds41_ple_global_scale.restype = C.c_float
    core.ds41_ple_global_scale.argtypes = [C.c_float]
    core.ds41_ple_convert.restype = C.c_int
    core.ds41_ple_convert.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_int]
    return core


def src_record_bytes(dim: int) -> int:
    return dim + dim // 32


def dst_record_bytes(dim: int) -> int:
    return dim // 2 + dim // 16


def scan_rows(rows_q: np.ndarray, dim: int = 256, threads: int = 8) -> float:
    """Largest magnitude of uint8 records [n, >= dim + dim/32]; NaN if any payload or scale byte encodes NaN."""
    assert rows_q.dtype == np.uint8 and rows_q.ndim == 2 and rows_q.flags.c_contiguous
    amax = C.c_float(0.0)
    rc = _core().ds41_ple_scan(rows_q.ctypes.data, rows_q.shape[0], dim, rows_q.shape[1], threads, C.byref(amax))
    if rc == 1:
        raise ValueError("bad table geometry")
    return float(amax.value)


def global_scale(amax: float) -> float:
    return float(_core().ds41_ple_global_scale(C.c_float(amax)))


def convert_rows(rows_q: np.ndarray, scale: float, dim: int = 256, threads: int = 8, out: np.ndarray | None = None):
    """uint8 FP8 records [n, >= dim + dim/32] -> uint8 NVFP4 records [n, dim/2 + dim/16] for the table scale `scale`."""
    assert rows_q.dtype == np.uint8 and rows_q.ndim == 2 and rows_q.flags.c_contiguous
    n = rows_q.shape[0]
    if out is None:
        out = np.empty((n, dst_record_bytes(dim)), dtype=np.uint8)
    assert out.dtype == np.uint8 and out.shape[0] == n and out.flags.c_contiguous and out.flags.writeable
    rc = _core().ds41_ple_convert(rows_q.ctypes.data, n, dim, rows_q.shape[1], C.c_float(scale), out.ctypes.data,
                                  out.shape[1], threads)
    if rc != 0:
        raise ValueError("bad table geometry or scale")
    return out


def _fingerprint(path: str) -> dict:
    st = os.stat(path)
    h = hashlib.blake2b(digest_size=16)
    with open(path, "rb") as f:
        h.update(f.read(1 << 20))
        if st.st_size > (2 << 20):
            f.seek(st.st_size - (1 << 20))
            h.update(f.read(1 << 20))
    return {"bytes": st.st_size, "mtime_ns": st.st_mtime_ns, "edges": h.hexdigest()}


def _write_json(path: str, doc: dict) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(doc, f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def convert_table(src: str, dst: str, rows: int, dim: int = 256, threads: int = 8, chunk_rows: int = 262144,
                  stop_after_chunks: int | None = None, log=None) -> dict:
    """Stream `src` (FP8 records) into `dst` (NVFP4 records); returns the metadata also written to `dst + ".json"`.
    `stop_after_chunks` ends the run early after that many newly finished chunks (the progress file then lets the next
    call continue); it exists for the resume test and for time-boxed runs."""
    sb, db = src_record_bytes(dim), dst_record_bytes(dim)
    if os.path.getsize(src) != rows * sb:
        raise ValueError(f"{src}: {os.path.getsize(src)} bytes, expected rows x {sb} = {rows * sb}")
    ident = {"source": _fingerprint(src), "rows": rows, "dim": dim, "chunk_rows": chunk_rows}
    prog_path, meta_path = dst + ".progress.json", dst + ".json"
    prog = {"identity": ident, "amax": None, "scanned_chunks": 0, "partial_amax": 0.0, "converted_chunks": 0}
    if os.path.exists(prog_path):
        with open(prog_path) as f:
            old = json.load(f)
        if old.get("identity") == ident:
            prog = old
    table = np.memmap(src, dtype=np.uint8, mode="r", shape=(rows, sb))
    n_chunks = (rows + chunk_rows - 1) // chunk_rows
    done_now, t0 = 0, time.time()

    def budget_spent():
        return stop_after_chunks is not None and done_now >= stop_after_chunks

    # pass 1: table amax
    while prog["scanned_chunks"] < n_chunks and not budget_spent():
        c = prog["scanned_chunks"]
        part = scan_rows(np.ascontiguousarray(table[c * chunk_rows:(c + 1) * chunk_rows]), dim, threads)
        if math.isnan(part):
            raise ValueError(f"{src}: NaN in records {c * chunk_rows}..{min(rows, (c + 1) * chunk_rows) - 1}")
        prog["partial_amax"] = max(prog["partial_amax"], part)
        prog["scanned_chunks"] = c + 1
        done_now += 1
        _write_json(prog_path, prog)
        if log:
            log(f"scan {c + 1}/{n_chunks} amax {prog['partial_amax']:.6g}")
    if prog["scanned_chunks"] < n_chunks:
        return {"complete": False, **prog}
    prog["amax"] = prog["partial_amax"]
    if not prog["amax"] > 0.0:
        raise ValueError(f"{src}: the table is all zeros")
    scale = global_scale(prog["amax"])
    # pass 2: records
    if not os.path.exists(dst) or os.path.getsize(dst) != rows * db:
        with open(dst, "wb") as f:
            f.truncate(rows * db)
        prog["converted_chunks"] = 0
    out = np.memmap(dst, dtype=np.uint8, mode="r+", shape=(rows, db))
    while prog["converted_chunks"] < n_chunks and not budget_spent():
        c = prog["converted_chunks"]
        lo, hi = c * chunk_rows, min(rows, (c + 1) * chunk_rows)
        convert_rows(np.ascontiguousarray(table[lo:hi]), scale, dim, threads, out=out[lo:hi])
        out.flush()
        prog["converted_chunks"] = c + 1
        done_now += 1
        _write_json(prog_path, prog)
        if log:
            log(f"convert {c + 1}/{n_chunks}")
    del out
    if prog["converted_chunks"] < n_chunks:
        return {"complete": False, **prog}
    meta = {"complete": True, "format": "nvfp4", "rows": rows, "dim": dim, "row_bytes": db, "global_scale": scale,
            "amax": prog["amax"], "source": ident["source"], "seconds": round(time.time() - t0, 3)}
    _write_json(meta_path, meta)
    return meta


def dequant_rows_reference(rows_q, scale: float, dim: int = 256):
    """uint8 NVFP4 records [n, >= dim/2 + dim/16] (torch tensor) -> fp32 [n, dim]: (code * block scale) * table scale."""
    import torch
    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
    payload = rows_q[:, :dim // 2].to(torch.int64)
    codes = torch.stack([payload & 15, payload >> 4], dim=-1).reshape(rows_q.shape[0], dim)
    sc = rows_q[:, dim // 2:dim // 2 + dim // 16].contiguous().view(torch.float8_e4m3fn).float()
    return (lut.to(rows_q.device)[codes] * sc.repeat_interleave(16, dim=1)) * scale


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--rows", type=int, required=True)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--threads", type=int, default=8)
    ap.add_argument("--chunk-rows", type=int, default=262144)
    args = ap.parse_args(argv)
    meta = convert_table(args.src, args.dst, args.rows, args.dim, args.threads, args.chunk_rows,
                         log=lambda m: print(m, flush=True))
    print(json.dumps(meta))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
