"""Decode sessions: CUDA-graph capture of the engine's per-step launch sequence and the public
generate loop.

`DecodeSession.generate()` is the user-facing call: prompt token ids in, generated ids out.  Each
decode step copies that step's inputs from pinned host memory, replays the captured graph and reads
the chosen tokens back (the tokens have to reach the host anyway to be streamed to a client).
`run_device_loop()` instead feeds the chosen token back on the device, so K steps are K graph replays
with no host round trip - the kernel-only number.

Reference behaviour being replaced: lazily captured per-shape CUDA graphs keyed by (rows, bindings)
(docs/ENGINEERING.md:23, rust/crates/ds41rt-daemon/src/v41_layer_graphs.rs).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..models.ds41 import DS41Engine
from ..ops import lib


class DecodeSession:
    def __init__(self, engine: DS41Engine, use_graphs: bool = True):
        self.e = engine
        self.use_graphs = use_graphs and engine.device.type == "cuda"
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.launches_per_graph: Dict[tuple, int] = {}
        R = engine.max_rows
        self.h_tokens = torch.zeros(R, dtype=torch.int32).pin_memory()
        self.h_pos = torch.zeros(R, dtype=torch.int32).pin_memory()
        self.h_slot = torch.full((R,), -1, dtype=torch.int32).pin_memory()
        self.h_chosen = torch.zeros(R, dtype=torch.int32).pin_memory()
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ graphs
    def _enqueue(self, rows: int, feedback: bool):
        self.e.forward_rows(rows)
        if feedback:
            self.e._run("feedback", self.e.k.ds41_decode_feedback, lib.ptr(self.e.chosen), lib.ptr(self.e.in_tokens),
                        lib.ptr(self.e.row_pos), rows, lib.stream())

    def graph(self, rows: int, feedback: bool = False) -> Optional[torch.cuda.CUDAGraph]:
        key = (rows, feedback)
        if not self.use_graphs:
            return None
        if key not in self.graphs:
            # one eager pass first: sets function attributes and warms every code path
            snapshot = (self.e.in_tokens.clone(), self.e.row_pos.clone())
            self._enqueue(rows, feedback)
            torch.cuda.synchronize()
            self.e.in_tokens.copy_(snapshot[0])
            self.e.row_pos.copy_(snapshot[1])
            before = self.e.launches
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue(rows, feedback)
            self.launches_per_graph[key] = self.e.launches - before
            self.e.in_tokens.copy_(snapshot[0])
            self.e.row_pos.copy_(snapshot[1])
            self.graphs[key] = g
        return self.graphs[key]

    # ------------------------------------------------------------------ stepping
    def step(self, tokens: List[int], positions: List[int], slots: List[int]) -> List[int]:
        """One pass through the public path: pinned H2D of the inputs, graph replay, D2H of the result."""
        n = len(tokens)
        e = self.e
        self.h_tokens[:n] = torch.tensor(tokens, dtype=torch.int32)
        self.h_pos[:n] = torch.tensor(positions, dtype=torch.int32)
        self.h_slot[:n] = torch.tensor(slots, dtype=torch.int32)
        e.in_tokens[:n].copy_(self.h_tokens[:n], non_blocking=True)
        e.row_pos[:n].copy_(self.h_pos[:n], non_blocking=True)
        e.row_slot[:n].copy_(self.h_slot[:n], non_blocking=True)
        self.h2d_bytes += 3 * 4 * n
        g = self.graph(n)
        if g is not None:
            g.replay()
        else:
            e.forward_rows(n)
        self.h_chosen[:n].copy_(e.chosen[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * n
        return self.h_chosen[:n].tolist()

    def run_device_loop(self, rows: int, steps: int):
        """`steps` decode steps with on-device token feedback (no host synchronisation inside)."""
        g = self.graph(rows, feedback=True)
        for _ in range(steps):
            if g is not None:
                g.replay()
            else:
                self._enqueue(rows, True)

    # ------------------------------------------------------------------ public generate
    def generate(self, prompt: List[int], max_new_tokens: int, slot: int = 0, eos: Optional[int] = None,
                 prefill_chunk: Optional[int] = None) -> List[int]:
        e = self.e
        assert e.cache.ensure(slot, len(prompt) + max_new_tokens + 1), "KV pool exhausted"
        nxt = e.prefill(slot, prompt, chunk=prefill_chunk)
        out = [nxt]
        pos = len(prompt)
        while len(out) < max_new_tokens and (eos is None or out[-1] != eos):
            out.append(self.step([out[-1]], [pos], [slot])[0])
            pos += 1
        e.check_status("generate")
        return out
