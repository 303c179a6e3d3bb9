"""Serving on several GPUs: rank 0 owns the HTTP server and the scheduler, the other ranks mirror its engine calls.

Every rank holds its shard of the model and runs the same launch sequence (the kernels meet in peer memory), so the
only thing the followers need is the sequence of engine calls with their host-side arguments.  `LeaderEngine` wraps the
rank-0 engine: each call that launches work (or changes the page tables) is first broadcast as a small message over a
CPU process group, then executed locally; `follower_loop` executes the same calls on the other ranks until it is told
to stop.  Collectives inside those calls (e.g. the vocabulary-shard gather of `logits_rows`) therefore line up.

The reference's counterpart is its coordinator / expert-worker split over TCP and RoCE
(rust/crates/ds41rt-daemon/src/v41_experts/coordinator.rs, service.rs:12-44); here all ranks are peers of one program.
"""
from __future__ import annotations

from typing import Any, List, Optional, Tuple


def make_control_group(fabric, timeout_s: float = 600.0):
    """A gloo group over the same ranks for host-side control messages (None on one rank).  Its collectives give up
    after `timeout_s`, so a leader whose follower vanished does not wait for ever."""
    if fabric.world == 1:
        return None
    import datetime
    import torch.distributed as dist
    return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))


def _bcast(group, obj: Any, src: int = 0) -> Any:
    import torch.distributed as dist
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


class _CacheMirror:
    def __init__(self, leader: "LeaderEngine"):
        self._l = leader

    def __getattr__(self, name):
        return getattr(self._l.eng.cache, name)

    def admit(self):
        self._l._send(("admit",))
        return self._l.eng.cache.admit()

    def ensure(self, slot: int, n_tokens: int) -> bool:
        self._l._send(("ensure", slot, n_tokens))
        return self._l.eng.cache.ensure(slot, n_tokens)

    def release(self, slot: int) -> None:
        self._l._send(("release", slot))
        self._l.eng.cache.release(slot)

    def snapshot(self, slot: int, n_tokens: int):
        self._l._sid += 1
        self._l._send(("snapshot", slot, n_tokens, self._l._sid))
        snap = self._l.eng.cache.snapshot(slot, n_tokens)
        snap.sid = self._l._sid
        return snap

    def restore_prefix(self, slot: int, snap, n_tokens: int) -> bool:
        self._l._send(("restore_prefix", slot, snap.sid, n_tokens))
        return self._l.eng.cache.restore_prefix(slot, snap, n_tokens)

    def restore(self, slot: int, snap) -> bool:
        self._l._send(("restore", slot, snap.sid))
        return self._l.eng.cache.restore(slot, snap)

    def drop_snapshot(self, snap) -> None:
        self._l._send(("drop", snap.sid))
        self._l.eng.cache.drop_snapshot(snap)


class LeaderEngine:
    """Drop-in for DS41Engine on rank 0 (the subset the serving backend uses)."""

    def __init__(self, engine, group, heartbeat=None):
        """heartbeat: parallel.health.Heartbeat of this rank (optional).  Its guard runs before every mirrored call -
        between passes, with nothing in flight - and raises RankFailure when a follower left or went silent."""
        self.eng, self.group, self.heartbeat = engine, group, heartbeat
        self._sid = 0
        self.cache = _CacheMirror(self)

    def __getattr__(self, name):
        return getattr(self.eng, name)

    def _send(self, msg: Tuple) -> None:
        if self.heartbeat is not None:
            self.heartbeat.guard()
        if self.group is None:
            return
        try:
            _bcast(self.group, msg)
        except RuntimeError:
            # A follower that left between the guard and this message closes its end of the control group.  The store
            # says who and why a moment later: report that (RankFailure) rather than the transport's error.
            if self.heartbeat is not None:
                import time
                deadline = time.time() + 5.0
                while time.time() < deadline and not self.heartbeat.peers_down():
                    time.sleep(0.05)
                self.heartbeat.guard()
            raise

    def set_rows(self, tokens: List[int], positions: List[int], slots: List[int], row_lo=None) -> None:
        self._send(("set_rows", list(tokens), list(positions), list(slots), None if row_lo is None else list(row_lo)))
        self.eng.set_rows(tokens, positions, slots, row_lo=row_lo)

    def forward_rows(self, rows: int, **kw) -> None:
        self._send(("forward", rows, kw))
        self.eng.forward_rows(rows, **kw)

    def ced_encoder_slice(self, c0: int, c1: int, r0: int, sources: bool = True) -> None:
        self._send(("ced_enc", c0, c1, r0, sources))
        self.eng.ced_encoder_slice(c0, c1, r0, sources)

    def ced_replay_slice(self, c0: int, c1: int, r0: int, head: bool) -> None:
        self._send(("ced_replay", c0, c1, r0, head))
        self.eng.ced_replay_slice(c0, c1, r0, head)

    def set_engram_rows(self, layer: int, rows_q, text_mask=None) -> None:
        """The leader's gathered table rows travel with the pass: every rank applies the same Engram update to its
        replicated streams."""
        import numpy as np
        arr = np.ascontiguousarray(rows_q.numpy() if hasattr(rows_q, "numpy") else rows_q)
        mask = None if text_mask is None else [int(m) for m in text_mask]
        self._send(("engram", layer, arr, mask))
        self.eng.set_engram_rows(layer, arr, mask)

    def clear_engram_rows(self) -> None:
        self._send(("engram_clear",))
        self.eng.clear_engram_rows()

    def logits_rows(self, rows: int):
        self._send(("logits", rows))
        return self.eng.logits_rows(rows)

    def check_status(self, what: str = "engine pass") -> None:
        self.eng.check_status(what)

    def stop_followers(self) -> None:
        self._send(("stop",))


def follower_loop(engine, group, on_error=None, heartbeat=None) -> int:
    """Run on ranks > 0 until the leader says stop; returns the number of passes executed.  A call that raises is
    reported (on_error) and, with a heartbeat, announced as this rank leaving: the leader's guard then fails its
    requests instead of waiting on kernels that never meet their peer."""
    passes = 0
    snaps = {}
    while True:
        msg = _bcast(group, None)
        op = msg[0]
        if op == "stop":
            return passes
        try:
            if op == "admit":
                engine.cache.admit()
                continue
            if op == "set_rows":
                engine.set_rows(msg[1], msg[2], msg[3], row_lo=msg[4])
            elif op == "forward":
                engine.forward_rows(msg[1], **msg[2])
                passes += 1
            elif op == "logits":
                engine.logits_rows(msg[1])
            elif op == "ced_enc":
                engine.ced_encoder_slice(msg[1], msg[2], msg[3], msg[4])
                passes += 1
            elif op == "ced_replay":
                engine.ced_replay_slice(msg[1], msg[2], msg[3], msg[4])
                passes += 1
            elif op == "engram":
                engine.set_engram_rows(msg[1], msg[2], msg[3])
            elif op == "engram_clear":
                engine.clear_engram_rows()
            elif op == "ensure":
                engine.cache.ensure(msg[1], msg[2])
            elif op == "release":
                engine.cache.release(msg[1])
            elif op == "snapshot":
                snaps[msg[3]] = engine.cache.snapshot(msg[1], msg[2])
            elif op == "restore":
                engine.cache.restore(msg[1], snaps[msg[2]])
            elif op == "restore_prefix":
                engine.cache.restore_prefix(msg[1], snaps[msg[2]], msg[3])
            elif op == "drop":
                engine.cache.drop_snapshot(snaps.pop(msg[1]))
        except Exception as e:          # keep the launch sequences aligned; the leader sees the status word / timeout
            if on_error is not None:
                on_error(e)
            if heartbeat is not None:
                heartbeat.leave(f"follower call {op} failed: {type(e).__name__}: {e}"[:200])
                return passes
