"""Two-stage pipeline parallelism over peer memory: the lower layers on one GPU, the upper layers and the vocabulary
head on another, the residual streams handed over at the boundary.

Each stage owns a DS41Engine that holds only its layers (EngineWeights(..., layer_range=...)).  What crosses the boundary
is the state before the boundary layer's hyper-connection step: the four residual streams, the last sublayer's expert
plane that is still to be merged, that sublayer's post / comb coefficients and the collapse weights - 5 small arrays
per pass.  The producer copies them into one of two slots of its symmetric buffer and raises its `sent` counter; the
consumer's pull kernel waits (bounded) on that counter through a peer pointer and copies the slot with plain peer
loads, then raises its own `consumed` counter so that the producer may reuse the slot two handoffs later.  Greedy
tokens travel the other way through the same mechanism, so a decode loop never leaves the GPUs.

With two slots the stages overlap on chunked prompts: stage 0 runs chunk k + 1 while stage 1 runs chunk k.

Reference: the dual-GPU layer split (layers 0-19 + embedding on one card, layers 20-39 + head on the other, residual
handoff by peer copy), docs/phase2-dual-rtx.md:57-66, rust/crates/ds41rt-daemon/src/v41_target_pass/distributed.rs:26-40,
rust/crates/ds41rt-daemon/src/v41_block/transfer.rs.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import lib

F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32


def slot_layout(max_rows: int, hidden: int, mult: int = 4):
    """Byte offsets of one handoff slot: streams bf16 [R, mult, H], plane f32 [R, H], post f32 [R, mult],
    comb f32 [R, mult * mult], pre f32 [R, mult]; every part starts on a 16-byte boundary."""
    sizes = [max_rows * mult * hidden * 2, max_rows * hidden * 4, max_rows * mult * 4, max_rows * mult * mult * 4,
             max_rows * mult * 4]
    offs, at = [], 0
    for n in sizes:
        offs.append(at)
        at += (n + 15) // 16 * 16
    return offs, sizes, at


def buffer_bytes(max_rows: int, hidden: int, mult: int = 4) -> int:
    """Symmetric bytes one stage needs: two slots, a token area and the four counters."""
    _, _, slot = slot_layout(max_rows, hidden, mult)
    return 2 * slot + (max_rows * 4 + 15) // 16 * 16 + 64


class PipelineStage:
    """One stage of a two-stage pipeline.  `stage` 0 owns layers [0, boundary), stage 1 owns [boundary, n_layers) and
    the head.  `my_buf` is this stage's symmetric buffer (uint8 tensor of buffer_bytes()), `peer_ptr` the device
    address of the other stage's buffer as seen from this GPU."""

    def __init__(self, engine, stage: int, boundary: int, my_buf: torch.Tensor, peer_ptr: int):
        cfg = engine.cfg
        assert stage in (0, 1) and 0 < boundary < engine.n_layers and engine.world == 1
        # the upper stage must not depend on caches or selections that only the lower stage holds
        for l in range(boundary, engine.n_layers):
            src, prod = cfg.source_of(l), cfg.index_producer_of(l)
            assert src is None or src >= boundary, f"layer {l} reads the compressed source of layer {src} (lower stage)"
            assert prod is None or prod >= boundary, f"layer {l} reuses the key selection of layer {prod} (lower stage)"
        assert not (cfg.candidate_layer >= 0 and cfg.candidate_topk_blocks > 0 and cfg.candidate_layer < boundary
                    and any(l > cfg.candidate_layer for l in cfg.index_layers if l >= boundary)), \
            "candidate blocks are chosen below the boundary and used above it"
        self.e, self.stage, self.B = engine, stage, boundary
        self.R, self.H, self.m = engine.max_rows, cfg.hidden, cfg.hc_mult
        self.offs, self.sizes, self.slot_bytes = slot_layout(self.R, self.H, self.m)
        self.tok_off = 2 * self.slot_bytes
        self.flag_off = self.tok_off + (self.R * 4 + 15) // 16 * 16
        assert my_buf.numel() >= self.flag_off + 64 and my_buf.dtype == torch.uint8
        self.buf, self.my_ptr, self.peer_ptr = my_buf, my_buf.data_ptr(), peer_ptr
        # counters (u32 each): [0] handoffs sent, [1] handoffs consumed, [2] token sets sent, [3] token sets consumed
        self.n_handoff = 0
        self.n_tokens = 0
        self.k = lib.kernels()

    # ---------------------------------------------------------------- addressing
    def _mine(self, off: int) -> C.c_void_p:
        return C.c_void_p(self.my_ptr + off)

    def _peer(self, off: int) -> C.c_void_p:
        return C.c_void_p(self.peer_ptr + off)

    def _flag(self, ptr_fn, idx: int) -> C.c_void_p:
        return ptr_fn(self.flag_off + 4 * idx)

    def _view(self, off: int, nbytes: int, dtype, shape):
        return self.buf[off: off + nbytes].view(dtype).view(*shape)

    # ---------------------------------------------------------------- stage 0: run the lower layers and hand over
    def run_lower(self, rows: int, embed: bool = True):
        """Rows described by engine.set_rows(): embedding + layers [0, boundary), then publish the boundary state."""
        assert self.stage == 0
        e, k, st = self.e, self.k, lib.stream
        pre_idx_before = None
        e.forward_rows(rows, embed=embed, head=False, last_layer=self.B)
        pre_idx_before = e._cur
        self.n_handoff += 1
        n = self.n_handoff
        base = (n & 1) * self.slot_bytes
        if n > 2:          # the slot was last used by handoff n - 2: wait until the peer has pulled it
            lib.check(k.ds41_pp_wait(self._flag(self._peer, 1), n - 2, lib.ptr(e.status), 500, st()), "pp_wait")
        R, H, m = self.R, self.H, self.m
        small = rows <= e.fused_rows
        post, comb = e.coef[e._ccur] if small else (e.post, e.comb)
        parts = [(e.streams, BF16, (R, m, H)), (e.moe_plane, F32, (R, H)), (post, F32, (R, m)),
                 (comb, F32, (R, m * m)), (e.pre[pre_idx_before], F32, (R, m))]
        for (src, dt, shape), off, nb in zip(parts, self.offs, self.sizes):
            self._view(base + off, nb, dt, shape)[:rows].copy_(src[:rows])
        lib.check(k.ds41_pp_signal(self._flag(self._mine, 0), n, st()), "pp_signal")
        e._pending = None

    def take_tokens(self, rows: int):
        """Stage 0: pull the greedy tokens of the peer's last head pass into the engine's token inputs (the next
        pass's positions and slots come from the host as usual)."""
        assert self.stage == 0
        self.n_tokens += 1
        e, k, st = self.e, self.k, lib.stream
        lib.check(k.ds41_pp_pull(self._peer(self.tok_off), lib.ptr(e.in_tokens), C.c_longlong((rows * 4 + 15) // 16 * 16),
                                 self._flag(self._peer, 2), self.n_tokens, lib.ptr(e.status), 510, st()), "pp_pull")
        lib.check(k.ds41_pp_signal(self._flag(self._mine, 3), self.n_tokens, st()), "pp_signal")

    # ---------------------------------------------------------------- stage 1: take over and run the upper layers
    def run_upper(self, rows: int, head: bool = True):
        """Rows described by engine.set_rows() (same rows as the producer's pass): pull the boundary state, merge the
        pending sublayer, run layers [boundary, n_layers) and, with `head`, the vocabulary head."""
        assert self.stage == 1
        e, k, st = self.e, self.k, lib.stream
        self.n_handoff += 1
        n = self.n_handoff
        base = (n & 1) * self.slot_bytes
        # one pull of the whole slot into this stage's own copy of it, then local copies into the engine's buffers
        lib.check(k.ds41_pp_pull(self._peer(base), self._mine(base), C.c_longlong(self.slot_bytes), self._flag(self._peer, 0), n,
                                 lib.ptr(e.status), 520, st()), "pp_pull")
        lib.check(k.ds41_pp_signal(self._flag(self._mine, 1), n, st()), "pp_signal")
        R, H, m = self.R, self.H, self.m
        small = rows <= e.fused_rows
        e._cur, e._ccur = 0, 0
        post, comb = e.coef[0] if small else (e.post, e.comb)
        parts = [(e.streams, BF16, (R, m, H)), (e.moe_plane, F32, (R, H)), (post, F32, (R, m)),
                 (comb, F32, (R, m * m)), (e.pre[0], F32, (R, m))]
        for (dst, dt, shape), off, nb in zip(parts, self.offs, self.sizes):
            dst[:rows].copy_(self._view(base + off, nb, dt, shape)[:rows])
        e.forward_rows(rows, embed=False, head=head, first_layer=self.B, pending=(e._moe_bases, 1, 1, 0))

    def give_tokens(self, rows: int, row0: int = 0):
        """Stage 1: publish the greedy tokens of rows [row0, row0 + rows) of the last head pass for the producer's next
        pass (after a prompt only its last row continues the sequence)."""
        assert self.stage == 1
        e, k, st = self.e, self.k, lib.stream
        self.n_tokens += 1
        n = self.n_tokens
        if n > 1:
            lib.check(k.ds41_pp_wait(self._flag(self._peer, 3), n - 1, lib.ptr(e.status), 530, st()), "pp_wait")
        self._view(self.tok_off, self.R * 4, I32, (self.R,))[:rows].copy_(e.chosen[row0:row0 + rows])
        lib.check(k.ds41_pp_signal(self._flag(self._mine, 2), n, st()), "pp_signal")


def make_stage(fabric, cfg, weights_fn, boundary: int, max_rows: int, **engine_kw) -> PipelineStage:
    """Two ranks of `fabric` (world 2): rank r becomes stage r.  `weights_fn(layer_range)` builds that stage's
    EngineWeights.  The engine itself runs with single-GPU semantics; only the handoff uses the fabric."""
    from ..models.ds41 import DS41Engine
    from .fabric import Fabric
    assert fabric.world == 2
    stage = fabric.rank
    rng = (0, boundary) if stage == 0 else (boundary, cfg.n_layers)
    eng = DS41Engine(cfg, weights_fn(rng), Fabric.single(fabric.device), max_rows=max_rows, **engine_kw)
    sym = fabric.alloc(buffer_bytes(max_rows, cfg.hidden, cfg.hc_mult))
    return PipelineStage(eng, stage, boundary, sym.local, sym.peer_ptrs[1 - stage])
