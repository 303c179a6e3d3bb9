"""Tracing: environment-filtered log targets, per-layer device timing and activation dumps.

`DS41_LOG` selects targets and levels, e.g. `DS41_LOG=timing,sampling=debug,lane_schedule` (a bare name means info).
Targets used in this package: timing, sampling, lane_schedule, draft_policy, host_cache, graph_capture, logit_trace,
activation_trace.  `DS41_ACTIVATION_TRACE_DIR` (+ optional `DS41_ACTIVATION_TRACE_POSITION`) makes the engine write the
residual streams after every layer for the rows at that position (all rows when no position is given).
`DS41_NVTX=1` puts every kernel launch of the engine into an NVTX range named after its kernel class.
Counterpart in the reference: the `tracing` targets and env filter (rust/crates/ds41rt-daemon/src/main.rs:66-68), per
layer CUDA events (`v41_target_pass.rs:142-146`) and the activation dump (`v41_target_pass.rs:348-357,482-484`).
"""
from __future__ import annotations

import logging
import os
from typing import Dict, List, Optional

_LEVELS = {"trace": 5, "debug": logging.DEBUG, "info": logging.INFO, "warn": logging.WARNING, "error": logging.ERROR}
_configured = False
_spec: Dict[str, int] = {}


def _configure():
    global _configured
    if _configured:
        return
    _configured = True
    for item in filter(None, (s.strip() for s in os.environ.get("DS41_LOG", "").split(","))):
        name, _, level = item.partition("=")
        _spec[name] = _LEVELS.get(level.lower(), logging.INFO) if level else logging.INFO
    if _spec:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s %(message)s"))
        root = logging.getLogger("ds41")
        root.addHandler(handler)
        root.propagate = False
        root.setLevel(logging.WARNING)


def target(name: str) -> logging.Logger:
    """Logger `ds41.<name>`; silent unless DS41_LOG names it."""
    _configure()
    log = logging.getLogger(f"ds41.{name}")
    log.setLevel(_spec.get(name, logging.WARNING))
    return log


def enabled(name: str, level: int = logging.INFO) -> bool:
    return target(name).isEnabledFor(level)


class LayerTimer:
    """CUDA events at the end of every layer of a pass; `layer_us()` after the pass gives device time per layer."""

    def __init__(self):
        self.events: List = []

    def begin(self):
        import torch
        self.events = [torch.cuda.Event(enable_timing=True)]
        self.events[0].record()

    def mark(self):
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.events.append(ev)

    def layer_us(self) -> List[float]:
        import torch
        torch.cuda.synchronize()
        return [a.elapsed_time(b) * 1e3 for a, b in zip(self.events[:-1], self.events[1:])]


class ActivationTrace:
    def __init__(self, directory: str, position: Optional[int] = None):
        self.dir, self.position = directory, position
        os.makedirs(directory, exist_ok=True)

    @staticmethod
    def from_env() -> Optional["ActivationTrace"]:
        d = os.environ.get("DS41_ACTIVATION_TRACE_DIR")
        if not d:
            return None
        p = os.environ.get("DS41_ACTIVATION_TRACE_POSITION")
        return ActivationTrace(d, int(p) if p else None)

    def dump(self, layer: int, streams, row_pos, rows: int):
        """Blocking copy of the rows' residual streams (debugging aid, never on in production)."""
        import torch
        pos = row_pos[:rows].tolist()
        for r, p in enumerate(pos):
            if self.position is None or p == self.position:
                torch.save(streams[r].float().cpu(), os.path.join(self.dir, f"layer{layer:02d}_pos{p}.pt"))
