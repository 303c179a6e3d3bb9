"""Front end of the sparse latent attention kernels.

`attend()` runs one pass of MQA attention over {window ring rows} U {selected compressed rows} for every row of a
pass.  The tensor-core kernel (csrc/kernels/attend_tc.cu: tcgen05 MMAs, accumulators in tensor memory, every head of
a row sharing each gathered key tile) serves head widths 512 and 128 with up to 64 local heads; other shapes, or
DS41_ATTN=legacy in the environment, go to the warp-MMA kernels of csrc/kernels/sparse_attn.cu.
Semantics: native/cuda/kernels/v41_sparse_attention.cu:89-381 of the reference.
"""
from __future__ import annotations

import ctypes as C
import os

from . import lib

KEYS_PER_TILE = 64


TC_MIN_ROWS = 17      # decode-sized passes over bf16 rows (a handful of rows, one key tile per CTA) stay on the warp-MMA kernel


def tc_usable(D: int, heads: int, rows: int = TC_MIN_ROWS, quantised: bool = False) -> bool:
    """Does the tensor-core kernel serve this pass?  DS41_ATTN=legacy / tc forces one kernel for every pass.
    Passes over FP8 / FP4 cache rows take it at every size: its gather warps expand a key tile once for all heads
    (5 rows x 640 keys: 0.023 ms against 0.055 ms)."""
    mode = os.environ.get("DS41_ATTN", "")
    if D not in (128, 512) or heads > 64 or mode == "legacy":
        return False
    return mode == "tc" or quantised or rows >= TC_MIN_ROWS


def attend(*, q, ldq, q_off, rows, heads, D, window, ring, row_pos, row_slot, win, comp_pool, sel, n_sel, k,
           page_table, max_pages, page_rows, inv_freq, rope_dim, scale, n_splits, part_o, part_ml, sink, out, ldo,
           kv_row_bytes=0, comp_row_bytes=0, row_hi=None, row_lo=None, status=None, impl=None):
    """Enqueue the attention of one pass on the current stream.  `impl`: None (pick), "tc" or "legacy"."""
    kern = lib.kernels()
    if impl is None:
        impl = "tc" if tc_usable(D, heads, rows, kv_row_bytes > 0) else "legacy"
    if impl == "legacy":
        return kern.ds41_attend_kv(
            lib.ptr(q), C.c_longlong(ldq), q_off, rows, heads, D, window, ring, lib.ptr(row_pos), lib.ptr(row_slot),
            lib.ptr(win), lib.ptr(comp_pool), lib.ptr(sel), lib.ptr(n_sel), k, lib.ptr(page_table), max_pages,
            page_rows, lib.ptr(inv_freq), rope_dim, C.c_float(scale), n_splits, lib.ptr(row_hi), lib.ptr(part_o),
            lib.ptr(part_ml), lib.ptr(sink), lib.ptr(out), C.c_longlong(ldo), kv_row_bytes, comp_row_bytes,
            lib.ptr(row_lo), lib.stream())
    a = lib.AttendArgs()
    a.q, a.ldq, a.q_off = lib.ptr(q), ldq, q_off
    a.rows, a.heads, a.D, a.window, a.ring = rows, heads, D, window, ring
    a.row_pos, a.row_slot, a.row_hi, a.row_lo = lib.ptr(row_pos), lib.ptr(row_slot), lib.ptr(row_hi), lib.ptr(row_lo)
    a.win, a.comp_pool, a.sel, a.n_sel, a.k = lib.ptr(win), lib.ptr(comp_pool), lib.ptr(sel), lib.ptr(n_sel), k
    a.page_table, a.max_pages, a.page_rows = lib.ptr(page_table), max_pages, page_rows
    a.inv_freq, a.rope_dim, a.scale = lib.ptr(inv_freq), rope_dim, scale
    a.n_splits, a.part_o, a.part_ml, a.sink = n_splits, lib.ptr(part_o), lib.ptr(part_ml), lib.ptr(sink)
    a.out, a.ldo, a.kv_row_bytes, a.comp_row_bytes = lib.ptr(out), ldo, kv_row_bytes, comp_row_bytes
    a.status = lib.ptr(status)
    return kern.ds41_attend_tc(C.byref(a), lib.stream())
