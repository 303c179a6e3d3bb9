"""Speculative decoding rounds: dSpark drafts a block, the target verifies it in one pass.

One round (all on the device, CUDA-graph capturable):
    draft pass -> drafts become the verification inputs -> target pass over [anchor, d1..d_{w-1}] ->
    drafter rings are fed from the target's taps -> accept rule + next-round inputs (spec_feedback)
Accept rule (rust/crates/ds41rt-core/src/dspark_verify.rs:18-52 of the reference): draft j is accepted while it
equals the target's own choice after draft j-1; the target's choice after the last accepted row is emitted as
the bonus token and becomes the next anchor.  Because every cache row is addressed by token position, rows of
rejected drafts are simply rewritten when their position is processed again - there is no separate commit.
`forced_accept >= 0` pins the accepted count per round (fixed acceptance schedule for benchmarking random
weights, where real acceptance is meaningless).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..models.ds41 import DS41Engine, I32
from ..models.dspark import DSparkDrafter
from ..ops import lib


class SpecSession:
    def __init__(self, target: DS41Engine, drafter: DSparkDrafter, forced_accept: int = -1, use_graphs: bool = True):
        self.t, self.d = target, drafter
        self.width = drafter.width
        self.forced = forced_accept
        self.use_graphs = use_graphs
        dev = target.device
        z = lambda n, dt=I32: torch.zeros(n, dtype=dt, device=dev)
        self.accepted, self.n_emitted, self.next_anchor = z(1), z(1), z(1)
        self.emitted = z(self.width)
        self.total = z(1, torch.int64)
        self.graph = None
        self.launches_per_round = 0
        self.h_out = torch.zeros(self.width + 2, dtype=torch.int32).pin_memory()
        self.h_conf = torch.zeros(self.width, dtype=torch.float32).pin_memory()
        self.last_confidence: List[float] = []      # sigmoid of the drafter's confidence head, one per draft row
        self.h_in = torch.zeros(1 + 2 * self.width, dtype=torch.int32).pin_memory()
        g = drafter.max_groups
        self.h_out_groups = torch.zeros(g * self.width, dtype=torch.int32).pin_memory()
        self.h_conf_groups = torch.zeros(g * self.width, dtype=torch.float32).pin_memory()
        self._host_state = None
        self.h2d_bytes = self.d2h_bytes = 0

    # ------------------------------------------------------------------ prompt
    def start(self, slot: int, prompt: List[int], max_new: int, chunk: Optional[int] = None) -> int:
        """Prefill the target (feeding the drafter's rings chunk by chunk) and prime round 0's inputs.
        Returns the first generated token (the anchor of round 0)."""
        t, d = self.t, self.d
        chunk = chunk or t.max_rows
        assert t.cache.ensure(slot, len(prompt) + max_new + 2 * self.width + 2), "KV pool exhausted"
        nxt = -1
        for c0 in range(0, len(prompt), chunk):
            part = prompt[c0:c0 + chunk]
            t.set_rows(part, list(range(c0, c0 + len(part))), [slot] * len(part))
            last = c0 + chunk >= len(prompt)
            t.forward_rows(len(part), head=last)
            d.feed(len(part))
            if last:
                nxt = int(t.chosen[t.last_head_row].item())
        self.prime(slot, nxt, len(prompt))
        return nxt

    def prime(self, slot: int, anchor: int, pos: int):
        w = self.width
        self.t.set_rows([anchor] + [0] * (w - 1), list(range(pos, pos + w)), [slot] * w)
        self.d.set_draft_rows(anchor, pos, slot)
        self.total.zero_()

    # ------------------------------------------------------------------ one round
    def _enqueue_round(self):
        t, d, k, w = self.t, self.d, lib.kernels(), self.width
        d.draft()
        t._run("drafts_to_inputs", k.ds41_copy_ints, lib.ptr(d.drafts), lib.ptr(t.in_tokens[1:]), w - 1, lib.stream())
        t.forward_rows(w)
        d.feed(w)
        t._run("spec_feedback", k.ds41_spec_feedback, lib.ptr(t.in_tokens), lib.ptr(t.chosen), w, self.forced,
               self.t.cfg.eos if self.forced < 0 else -1, lib.ptr(self.accepted), lib.ptr(self.emitted),
               lib.ptr(self.n_emitted), lib.ptr(self.next_anchor), lib.ptr(t.row_pos), lib.ptr(d.eng.row_pos),
               lib.ptr(d.eng.row_hi), lib.ptr(t.in_tokens), lib.ptr(d.eng.in_tokens), lib.ptr(self.total),
               lib.stream())

    def round(self):
        if not self.use_graphs:
            self._enqueue_round()
            return
        if self.graph is None:
            snap = [x.clone() for x in (self.t.in_tokens, self.t.row_pos, self.d.eng.in_tokens, self.d.eng.row_pos,
                                        self.d.eng.row_hi, self.total)]
            self._enqueue_round()          # eager warm-up (sets kernel attributes)
            torch.cuda.synchronize()
            restore = lambda: [dst.copy_(src) for dst, src in zip(
                (self.t.in_tokens, self.t.row_pos, self.d.eng.in_tokens, self.d.eng.row_pos, self.d.eng.row_hi,
                 self.total), snap)]
            restore()
            before = self.t.launches + self.d.eng.launches
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue_round()
            self.launches_per_round = self.t.launches + self.d.eng.launches - before
            restore()
            self.graph = g
        self.graph.replay()

    def round_host(self, feed_inputs: bool = False) -> List[int]:
        """One round through the public path: (optionally) copy this round's anchor and positions from pinned
        host memory, replay, then read the emitted tokens back to pinned host memory."""
        w = self.width
        if feed_inputs and self._host_state is not None:
            anchor, pos = self._host_state
            self.h_in[0] = anchor
            self.h_in[1: 1 + w] = torch.arange(pos, pos + w, dtype=torch.int32)
            self.h_in[1 + w: 1 + 2 * w] = pos + w - 1
            t, e = self.t, self.d.eng
            t.in_tokens[0:1].copy_(self.h_in[0:1], non_blocking=True)
            e.in_tokens[0:1].copy_(self.h_in[0:1], non_blocking=True)
            t.row_pos[:w].copy_(self.h_in[1: 1 + w], non_blocking=True)
            e.row_pos[:w].copy_(self.h_in[1: 1 + w], non_blocking=True)
            e.row_hi[:w].copy_(self.h_in[1 + w: 1 + 2 * w], non_blocking=True)
            self.h2d_bytes += 4 * (2 + 3 * w)
        self.round()
        self.h_out[:w].copy_(self.emitted, non_blocking=True)
        self.h_out[w: w + 1].copy_(self.n_emitted, non_blocking=True)
        self.h_out[w + 1: w + 2].copy_(self.t.row_pos[0:1], non_blocking=True)
        self._read_confidence()
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * (w + 2)
        self._publish_confidence()
        n = int(self.h_out[w])
        toks = self.h_out[:n].tolist()
        self._host_state = (toks[-1], int(self.h_out[w + 1]))
        return toks

    # ------------------------------------------------------------------ host-selected rounds
    def draft_host(self, slot: int, anchor: int, pos: int) -> List[int]:
        """Draft pass alone: [anchor, noise...] at positions pos.. -> the width - 1 proposed tokens, on the host.
        For rounds whose verification rows are selected under masks or drawn by the sampler (the caller cuts the
        proposal, builds the row masks and then calls verify_host)."""
        w = self.width
        self.d.set_draft_rows(anchor, pos, slot)
        self.d.draft()
        self.h_out[: w - 1].copy_(self.d.drafts[: w - 1], non_blocking=True)
        self._read_confidence()
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * (w - 1)
        self._publish_confidence()
        return self.h_out[: w - 1].tolist()

    def draft_host_groups(self, slots: List[int], anchors: List[int], positions: List[int]):
        """One draft pass for several sequences -> (proposals, confidences): per sequence the width - 1 proposed tokens
        and the sigmoid of the confidence head per draft row ([] without a confidence head)."""
        w, g = self.width, len(slots)
        self.d.set_draft_rows_groups(anchors, positions, slots)
        self.d.draft(g)
        self.h_out_groups[: g * w].copy_(self.d.drafts[: g * w], non_blocking=True)
        if self.d.conf_w is not None:
            self.h_conf_groups[: g * w].copy_(self.d.confidence[: g * w], non_blocking=True)
            self.d2h_bytes += 4 * g * w
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * g * w
        toks = self.h_out_groups[: g * w].tolist()
        conf = torch.sigmoid(self.h_conf_groups[: g * w]).tolist() if self.d.conf_w is not None else []
        return ([toks[i * w: i * w + w - 1] for i in range(g)],
                [conf[i * w: (i + 1) * w] if conf else [] for i in range(g)])

    def verify_host_groups(self, slots: List[int], inputs: List[List[int]], positions: List[int]) -> List[int]:
        """One target pass over the verification rows of several sequences, back to back; returns the first row of
        each sequence in the pass.  The drafter's rings of every slot are fed from the target's taps."""
        toks, pos, sl, first = [], [], [], []
        for s, inp, p in zip(slots, inputs, positions):
            first.append(len(toks))
            toks += inp
            pos += list(range(p, p + len(inp)))
            sl += [s] * len(inp)
        self.t.set_rows(toks, pos, sl)
        self.t.forward_rows(len(toks))
        self.d.feed(len(toks))
        return first

    def _read_confidence(self):
        if self.d.conf_w is not None:
            self.h_conf.copy_(self.d.confidence[: self.width], non_blocking=True)
            self.d2h_bytes += 4 * self.width

    def _publish_confidence(self):
        if self.d.conf_w is not None:
            self.last_confidence = torch.sigmoid(self.h_conf).tolist()

    def verify_host(self, slot: int, inputs: List[int], pos: int) -> None:
        """Target pass over [anchor, drafts...] at positions pos..; the logits of every row stay in the engine and the
        drafter's rings are fed from the target's taps of these rows (a rejected row is rewritten when its position
        comes again)."""
        n = len(inputs)
        self.t.set_rows(inputs, list(range(pos, pos + n)), [slot] * n)
        self.t.forward_rows(n)
        self.d.feed(n)

    def generate(self, prompt: List[int], max_new_tokens: int, slot: int = 0, eos: Optional[int] = None) -> List[int]:
        first = self.start(slot, prompt, max_new_tokens)
        out = [first]
        while len(out) < max_new_tokens and (eos is None or eos not in out):
            out.extend(self.round_host())
        self.t.check_status("speculative generate (target)")
        self.d.eng.check_status("speculative generate (drafter)")
        if eos is not None and eos in out:
            out = out[: out.index(eos) + 1]
        return out[:max_new_tokens]
