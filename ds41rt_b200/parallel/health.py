"""Rank liveness over the rendezvous store: heartbeats, failure notes and a pre-launch guard.

Kernels that wait on a peer are bounded and report through a status word, but a second of spinning per launch is a
poor failure detector.  Every rank therefore publishes a heartbeat (and, when it fails, a note saying why) in a
key-value store that lives on the host; `guard()` is called between steps - never with a collective in flight - and
raises `RankFailure` before the next launch if a peer has left or gone silent.  A rank that wants to leave posts its
note first and only then stops launching.

The reference detects lost expert workers with per-phase transport timeouts and executor-id namespaces
(rust/crates/ds41rt-transport/src/v41_expert/roce.rs:12-22, v41_expert.rs:42-56) and fails the active requests while
the server keeps running (rust/crates/ds41rt-daemon/src/v41_native_serve/scheduler.rs:439-448).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], reasons: Dict[int, str]):
        self.ranks, self.reasons = ranks, reasons
        super().__init__("ranks unavailable: " + ", ".join(f"{r} ({reasons.get(r, 'silent')})" for r in ranks))


class DictStore:
    """In-process stand-in for a distributed store (tests, single-process use)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    """`store` needs set/get/check (torch.distributed.TCPStore, FileStore, or DictStore)."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.2, max_age: float = 2.0,
                 clock=time.time, prefix: str = "ds41/hb", join_grace: float = 10.0):
        """`join_grace`: how long after this rank's own start a peer may still be without its first beat before it
        counts as "never joined" (ranks leave their rendezvous at slightly different times)."""
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.max_age, self.clock, self.prefix = interval, max_age, clock, prefix
        self.join_grace = join_grace
        self._born = clock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.beat()

    # ------------------------------------------------------------------ publishing
    def beat(self) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", repr(self.clock()))

    def start(self) -> "Heartbeat":
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, name="ds41-heartbeat", daemon=True)
        self._thread.start()
        return self

    def wait_joined(self, timeout: float = 30.0) -> bool:
        """Block until every peer has posted its first beat (or `timeout` real seconds pass)."""
        keys = [f"{self.prefix}/{r}" for r in range(self.world) if r != self.rank]
        deadline = time.time() + timeout
        while time.time() < deadline:
            try:
                if self.store.check(keys):
                    return True
            except Exception:
                return False
            time.sleep(min(0.05, self.interval))
        return False

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def leave(self, reason: str) -> None:
        """Announce that this rank stops launching (call it between steps, then stop)."""
        try:
            self.store.set(f"{self.prefix}/left/{self.rank}", reason)
        finally:
            self.stop()

    # ------------------------------------------------------------------ checking
    def peers_down(self) -> Dict[int, str]:
        """Peers that left, never joined or went silent.  A store that cannot be reached counts as a failure too: the
        rank that hosts it is gone (or the network to it is), so every peer is reported with that reason."""
        now, down = self.clock(), {}
        try:
            for r in range(self.world):
                if r == self.rank:
                    continue
                if self.store.check([f"{self.prefix}/left/{r}"]):
                    down[r] = self.store.get(f"{self.prefix}/left/{r}").decode()
                    continue
                key = f"{self.prefix}/{r}"
                if not self.store.check([key]):
                    if now - self._born >= self.join_grace:
                        down[r] = "never joined"
                    continue
                age = now - float(self.store.get(key).decode())
                if age > self.max_age:
                    down[r] = f"silent for {age:.1f} s"
        except Exception as e:           # TCPStore raises DistNetworkError / RuntimeError when its host is gone
            why = f"store unreachable: {type(e).__name__}"
            for r in range(self.world):
                if r != self.rank:
                    down.setdefault(r, why)
        return down

    def guard(self) -> None:
        """Raise before a launch that would wait on a rank that is gone."""
        down = self.peers_down()
        if down:
            raise RankFailure(sorted(down), down)
