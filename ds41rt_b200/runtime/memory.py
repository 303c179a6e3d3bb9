"""Start-up memory plan of the serving process: how many KV pages fit beside the weights.

One page covers `page_tokens` positions of every compressed source (rows = page_tokens / ratio per source, each a KV row
plus an index-key row).  The pool wants  ceil(ctx / page_tokens) * (slots + 2) + slots + 2 * retained  pages - every slot
at full context, two spare contexts for snapshots in flight, one partial page per slot and two per retained snapshot -
and is cut to what the device has free after the weights, minus a fixed headroom.  The window rings (layers x slots x
ring rows) and the step buffers are accounted before the pool.
Reference: rust/crates/ds41rt-daemon/src/v41_native_serve/memory.rs:9-13,137-204,354-370 (page groups, pool plan).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from ..config import ModelConfig
from . import core as K

HEADROOM_BYTES = 2 << 30


@dataclass
class PoolPlan:
    page_tokens: int
    bytes_per_page: int
    pages_wanted: int
    pages: int
    pool_bytes: int
    ring_bytes: int
    budget_bytes: int
    tokens: int
    limited_by_memory: bool

    def as_dict(self) -> dict:
        return asdict(self)


def kv_row_bytes(cfg: ModelConfig, kv_dtype: str) -> tuple:
    """(window row bytes, compressed row bytes) of one latent row."""
    D = cfg.head_dim
    if kv_dtype == "bf16":
        return 2 * D, 2 * D
    fp8 = (D + D // 32 + 15) // 16 * 16
    if kv_dtype == "fp8":
        return fp8, fp8
    return fp8, (D // 2 + D // 16 + 15) // 16 * 16


def plan_pool(cfg: ModelConfig, *, n_layers: int, slots: int, max_context: int, free_bytes: int, kv_dtype: str = "bf16",
              page_tokens: int = 64, retained: int = 40, ring_rows: Optional[int] = None,
              reserve_bytes: int = 0) -> PoolPlan:
    win_row, comp_row = kv_row_bytes(cfg, kv_dtype)
    per_page = 0
    for src, ratio in cfg.source_layers.items():
        if src < n_layers:
            per_page += (page_tokens // ratio) * (comp_row + 2 * cfg.index_dim)
    ring = ring_rows if ring_rows is not None else cfg.window + 16
    ring_bytes = n_layers * slots * ring * win_row
    budget = max(0, free_bytes - ring_bytes - reserve_bytes - HEADROOM_BYTES)
    wanted = (max_context + page_tokens - 1) // page_tokens * (slots + 2) + slots + 2 * retained
    pages = wanted if per_page == 0 else K.plan_kv_groups(max_context, page_tokens, slots, retained, per_page, budget)
    pages = max(0, int(pages))
    return PoolPlan(page_tokens, per_page, wanted, pages, pages * per_page, ring_bytes, budget, pages * page_tokens,
                    pages < wanted)
