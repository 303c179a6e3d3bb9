"""dSpark drafter: a few DS41 blocks that propose a block of draft tokens per round.

Structure (reference: architecture.md:62-66, rust/crates/ds41rt-daemon/src/v41_experts/dspark/main_context.rs:1-60,
native/cuda/kernels/v41_dspark.cu:40-58,241-290):
  * conditioning: the means of the target's residual streams entering its tap layers are concatenated, projected by
    `mtp.0.main_proj` and normalised (`main_norm`); every drafter stage turns those rows into committed KV
    (its own wkv / kv_norm / plain RoPE) stored in a position-indexed ring of 128 rows;
  * a draft pass feeds [anchor token, noise, noise, ...] through the stages; draft rows attend to the ring and to
    each other without a causal mask; stages have their own mHC, attention and a smaller MoE;
  * terminal: final norm, the TARGET's vocabulary head, plus a low-rank Markov head whose bias is chained position
    by position (token j conditions the logits of token j+1); greedy selection.
The drafter blocks are executed by a second DS41Engine instance that shares the target's embedding/head tensors.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig
from ..ops import gemm as G
from ..ops import lib
from .ds41 import BF16, DS41Engine, EngineWeights, F32, I32


def drafter_config(cfg: ModelConfig) -> ModelConfig:
    d = cfg.dspark
    return dataclasses.replace(cfg, name=cfg.name + "-dspark", n_layers=d.stages, compress_ratios=[0] * d.stages,
                               source_layers={}, index_layers=(), n_experts=d.n_experts, topk=d.topk,
                               window=d.ring_rows, dspark=None, engram=None, vision=None)


class DSparkDrafter:
    def __init__(self, cfg: ModelConfig, target: DS41Engine, weights: Optional[Dict[str, torch.Tensor]] = None,
                 width: Optional[int] = None, seed: int = 0, expert_dtype: str = "bf16", max_groups: int = 4):
        """`max_groups`: how many sequences one draft pass can serve (each gets its own block of `width` rows, its own
        slot's rings and its own Markov chain)."""
        assert cfg.dspark is not None
        d = cfg.dspark
        self.cfg, self.target, self.d = cfg, target, d
        self.width = width or d.block_size
        self.max_groups = max(1, min(max_groups, target.max_rows // self.width, target.cache.slots))
        dev, rank, world = target.device, target.rank, target.world
        dcfg = drafter_config(cfg)
        H = cfg.hidden
        n_taps = len(d.tap_layers)
        last = d.stages - 1
        if weights is not None:
            ew = EngineWeights.from_fp32(dcfg, weights, rank, world, dev, prefix="mtp", n_layers=d.stages,
                                         n_experts=d.n_experts, topk=d.topk, share=target.w,
                                         expert_dtype=expert_dtype)
            to = lambda t, dt=BF16: t.to(device=dev, dtype=dt).contiguous()
            ew.final_norm = to(weights[f"mtp.{last}.norm.weight"], F32)
            self.main_proj = to(weights["mtp.0.main_proj.weight"])
            self.main_norm = to(weights["mtp.0.main_norm.weight"], F32)
            self.markov_embed = to(weights[f"mtp.{last}.markov_head.embed.weight"])
            v0 = rank * target.V_local
            self.markov_head = to(weights[f"mtp.{last}.markov_head.head.weight"][v0:v0 + target.V_local])
            conf = weights.get(f"mtp.{last}.confidence_head.proj.weight")
            self.conf_w = to(conf.reshape(-1)) if conf is not None else None
        else:
            ew = EngineWeights.random(dcfg, rank, world, dev, seed=seed + 77, share=target.w,
                                      expert_dtype=expert_dtype)
            gen = torch.Generator(device=dev).manual_seed(seed + 78)
            rnd = lambda *shape: (torch.randn(*shape, generator=gen, device=dev) * 0.02).to(BF16)
            self.main_proj = rnd(H, n_taps * H)
            self.main_norm = torch.ones(H, dtype=F32, device=dev)
            self.markov_embed = rnd(cfg.vocab, d.markov_rank)
            self.markov_head = rnd(target.V_local, d.markov_rank)
            self.conf_w = rnd(H + d.markov_rank)
        R = max(target.max_rows, self.width)
        self.eng = DS41Engine(dcfg, ew, target.fabric, max_rows=R, slots=target.cache.slots, max_ctx=64,
                              row_hi=True)
        self.eng.layer_prefix_plain = True
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
        self.taps_bf16 = z((R, n_taps * H), BF16)
        self.main_splits = G.pick_splits(H, n_taps * H, max_splits=16)
        self.main_planes = z((16, R, H), F32)
        self.n_blocks = 444          # three resident blocks per SM (markov_step is sized for it)
        self.block_val = z((self.n_blocks,), F32)
        self.block_idx = z((self.n_blocks,), I32)
        self.ticket = z((1,), I32)
        # group g owns entries [g * width, (g + 1) * width): drafts[g * width + j] = proposed token for position p_g + 1 + j
        self.drafts = z((self.max_groups * self.width,), I32)
        self.draft_val = z((self.max_groups * self.width,), F32)
        # raw confidence-head output per draft row (sigmoid on the host)
        self.confidence = z((self.max_groups * self.width,), F32)
        self.launches = 0

    # ------------------------------------------------------------------ conditioning
    def feed(self, rows: int):
        """Turn the target's tap means of its last pass (rows/positions/slots as in the target's inputs)
        into committed ring rows of every drafter stage."""
        t, e, k = self.target, self.eng, lib.kernels()
        H = self.cfg.hidden
        n_taps = t.taps.shape[0]
        e._run("taps_pack", k.ds41_taps_pack, lib.ptr(t.taps), lib.ptr(self.taps_bf16), n_taps, rows, H,
               C.c_longlong(t.taps.stride(0)), lib.stream())
        e._run("gemm_main", G.linear_planes, self.taps_bf16[:rows], self.main_proj,
               self.main_planes.view(-1)[: self.main_splits * rows * H].view(self.main_splits, rows, H),
               self.main_splits, status=e.status)
        e._run("norm_main", k.ds41_norm_rows, lib.ptr(self.main_planes), self.main_splits, C.c_longlong(rows * H),
               lib.ptr(self.main_norm), lib.ptr(e.xn), rows, H, C.c_float(self.cfg.norm_eps), lib.stream())
        # the drafter engine's row metadata mirrors the target's
        e._run("copy_pos", k.ds41_copy_ints, lib.ptr(t.row_pos), lib.ptr(e.row_pos), rows, lib.stream())
        e._run("copy_slot", k.ds41_copy_ints, lib.ptr(t.row_slot), lib.ptr(e.row_slot), rows, lib.stream())
        e.feed_rings(rows)

    # ------------------------------------------------------------------ drafting
    def set_draft_rows(self, anchor: int, pos: int, slot: int):
        w = self.width
        toks = [anchor] + [self.d.noise_token_id] * (w - 1)
        self.eng.set_rows(toks, list(range(pos, pos + w)), [slot] * w, row_hi=[pos + w - 1] * w)

    def set_draft_rows_groups(self, anchors: List[int], positions: List[int], slots: List[int]):
        """One block of `width` rows per sequence, back to back: [anchor, noise, ...] at positions pos.. in its slot."""
        w = self.width
        assert 1 <= len(anchors) <= self.max_groups and len(set(slots)) == len(slots)
        toks, pos, sl, hi = [], [], [], []
        for a, p, s in zip(anchors, positions, slots):
            toks += [a] + [self.d.noise_token_id] * (w - 1)
            pos += list(range(p, p + w))
            sl += [s] * w
            hi += [p + w - 1] * w
        self.eng.set_rows(toks, pos, sl, row_hi=hi)

    def set_sampling(self, temperature: float = 0.0, seed: int = 0, subsequence: int = 0, offset: int = 0):
        """Draft tokens are sampled (Gumbel-max with Philox numbers) when temperature > 0, greedy otherwise.  `offset`
        is the first Philox counter of this draft pass; row j uses the block starting at offset + j * ceil(vocab/4)
        (reserve width * ceil(vocab/4) counters per pass, e.g. with runtime.core.DraftRng)."""
        self.sampling = (float(temperature), int(seed), int(subsequence), int(offset))

    def _draft_rng(self, j: int):
        import ctypes as C
        t, seed, sub, off = getattr(self, "sampling", (0.0, 0, 0, 0))
        if t <= 0.0:
            return None
        r = lib.DraftRng(t, seed & (2 ** 64 - 1), sub, off + j * ((self.cfg.vocab + 3) // 4))
        self._rng_keep = getattr(self, "_rng_keep", [])[-16:] + [r]
        return C.byref(r)

    def draft(self, groups: int = 1):
        """One draft pass over the rows prepared in the drafter engine's inputs (`groups` blocks of `width` rows) ->
        self.drafts (device).  The Markov chain runs position by position inside every block."""
        e, k, t = self.eng, lib.kernels(), self.target
        w = self.width
        assert 1 <= groups <= self.max_groups
        e.forward_rows(groups * w, head=False)
        e.head_logits(groups * w)
        rank = self.d.markov_rank
        for j in range(w):
            for g in range(groups):
                r = g * w + j                                    # row of the pass, entry of drafts
                prev = e.in_tokens[r:r + 1] if j == 0 else self.drafts[r - 1:r]
                e._run("markov_step", k.ds41_markov_step, lib.ptr(e.logits[r]), lib.ptr(self.markov_head),
                       lib.ptr(self.markov_embed), lib.ptr(prev), e.V_local, e.rank * e.V_local, rank, self.cfg.vocab,
                       lib.ptr(self.block_val), lib.ptr(self.block_idx), self.n_blocks, lib.ptr(self.ticket),
                       lib.ptr(e.best_val[r:r + 1]), lib.ptr(e.best_idx[r:r + 1]), self._draft_rng(r), lib.stream())
                if e.world > 1:
                    e._signal()
                    e._run("draft_merge", k.ds41_argmax_merge, _offset_ptrs(e._val_ptrs, 4 * r, e.world),
                           _offset_ptrs(e._idx_ptrs, 4 * r, e.world), e.world, 1, lib.ptr(self.drafts[r:r + 1]),
                           lib.ptr(e.flag_ptrs), lib.ptr(e.epoch), lib.ptr(e.status), lib.stream())
                else:
                    e._run("draft_take", k.ds41_copy_ints, lib.ptr(e.best_idx[r:r + 1]), lib.ptr(self.drafts[r:r + 1]),
                           1, lib.stream())
        if self.conf_w is not None:
            # collapsed (pre-norm) rows of the last stage and the Markov embedding each position was conditioned on
            for g in range(groups):
                r = g * w
                e._run("confidence", k.ds41_dspark_confidence, lib.ptr(e.xc[r:]), C.c_longlong(self.cfg.hidden),
                       lib.ptr(self.markov_embed), rank, lib.ptr(e.in_tokens[r:r + 1]), lib.ptr(self.drafts[r:]),
                       lib.ptr(self.conf_w), lib.ptr(self.confidence[r:]), w, self.cfg.hidden, self.cfg.vocab,
                       lib.stream())


def _offset_ptrs(ptrs, offset_bytes: int, n: int):
    return (C.c_void_p * n)(*[(p or 0) + offset_bytes for p in ptrs])
