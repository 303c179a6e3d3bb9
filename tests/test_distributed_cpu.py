"""Multi-rank serving, host side: the leader's engine calls reach the followers in order over the gloo control group, and
a follower whose call fails announces that it leaves, so that the leader's next call raises instead of launching kernels
that would wait for a missing peer.  Engines are recording fakes; no GPU is involved."""
import multiprocessing as mp
import os

import pytest

from ds41rt_b200.parallel.health import Heartbeat, RankFailure


class _FakeSnap:
    def __init__(self, sid=0):
        self.sid = sid


class _FakeCache:
    def __init__(self, log):
        self.log = log

    def admit(self):
        self.log.append(("admit",))
        return (0, 1)

    def ensure(self, slot, n):
        self.log.append(("ensure", slot, n))
        return True

    def release(self, slot):
        self.log.append(("release", slot))

    def snapshot(self, slot, n):
        self.log.append(("snapshot", slot, n))
        return _FakeSnap()

    def restore_prefix(self, slot, snap, n):
        self.log.append(("restore_prefix", slot, n))
        return True

    def restore(self, slot, snap):
        self.log.append(("restore", slot))
        return True

    def drop_snapshot(self, snap):
        self.log.append(("drop",))


class _FakeEngine:
    def __init__(self, fail_on_forward=-1):
        self.log = []
        self.cache = _FakeCache(self.log)
        self.fail_on_forward, self.forwards = fail_on_forward, 0

    def set_rows(self, tokens, positions, slots, row_lo=None):
        self.log.append(("set_rows", list(tokens), list(positions), list(slots), row_lo))

    def forward_rows(self, rows, **kw):
        self.forwards += 1
        if self.forwards == self.fail_on_forward:
            raise RuntimeError("device status 2 at site 201")
        self.log.append(("forward", rows, kw))

    def ced_encoder_slice(self, c0, c1, r0, sources=True):
        self.log.append(("ced_enc", c0, c1, r0, sources))

    def ced_replay_slice(self, c0, c1, r0, head):
        self.log.append(("ced_replay", c0, c1, r0, head))

    def set_engram_rows(self, layer, rows_q, text_mask=None):
        self.log.append(("engram", layer, bytes(rows_q.tobytes()), text_mask))

    def clear_engram_rows(self):
        self.log.append(("engram_clear",))

    def logits_rows(self, rows):
        self.log.append(("logits", rows))

    def check_status(self, what=""):
        pass


def _script(eng):
    """The calls of one request as the serving backend issues them."""
    import numpy as np
    eng.cache.admit()
    eng.cache.ensure(0, 96)
    eng.set_rows([5, 6, 7], [0, 1, 2], [0, 0, 0])
    eng.set_engram_rows(1, np.arange(12, dtype=np.uint8).reshape(3, 4), [1, 1, 0])
    eng.forward_rows(3, head=True)
    eng.clear_engram_rows()
    snap = eng.cache.snapshot(0, 3)
    eng.logits_rows(1)
    eng.set_rows([9], [3], [0], row_lo=[0])
    eng.forward_rows(1)
    eng.ced_encoder_slice(0, 64, 32, True)
    eng.ced_replay_slice(32, 64, 32, True)
    eng.cache.restore_prefix(1, snap, 2)
    eng.cache.restore(1, snap)
    eng.cache.drop_snapshot(snap)
    eng.cache.release(0)


def _rank(rank, world, port, store_port, fail, q):
    import torch.distributed as dist
    from ds41rt_b200.serving.distributed import LeaderEngine, follower_loop, make_control_group
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=False)
    hb = Heartbeat(store, rank, world, interval=0.05, max_age=5.0).start()
    hb.wait_joined(30.0)

    class _Fabric:
        pass
    fabric = _Fabric()
    fabric.world = world
    group = make_control_group(fabric, timeout_s=20.0)
    out = None
    try:
        if rank == 0:
            eng = _FakeEngine()
            lead = LeaderEngine(eng, group, heartbeat=hb)
            try:
                _script(lead)
                if fail:
                    import time
                    deadline = time.time() + 10.0
                    while time.time() < deadline:            # the follower's note arrives within a beat or two
                        time.sleep(0.1)
                        lead.set_rows([1], [4], [0])
                    out = ("no failure seen", eng.log)
                else:
                    lead.stop_followers()
                    out = ("ok", eng.log)
            except RankFailure as e:
                out = ("rank failure", e.ranks, dict(e.reasons))
        else:
            eng = _FakeEngine(fail_on_forward=2 if fail and rank == 1 else -1)
            errors = []
            passes = follower_loop(eng, group, on_error=errors.append, heartbeat=hb)
            out = ("follower", passes, eng.log, [str(e) for e in errors])
    except Exception as e:                                   # reported, not left to hang the parent
        out = ("error", f"{type(e).__name__}: {e}")
    q.put((rank, out))
    hb.stop()
    import time
    time.sleep(0.5)                                          # let the queue's feeder thread hand the result over
    os._exit(0)                                              # no collective teardown with a peer that may be gone


def _free_port():
    import random
    import socket
    for _ in range(200):
        port = random.randint(20000, 29999)
        with socket.socket() as s:
            try:
                s.bind(("127.0.0.1", port))
            except OSError:
                continue
        return port
    raise RuntimeError("no free port")


def _run(world, fail):
    import torch.distributed as dist
    host = dist.TCPStore("127.0.0.1", 0, None, is_master=True, wait_for_workers=False)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, world, port, host.port, fail, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world if not fail else 2):            # a failed run: the leader and the failing follower report
            rank, out = q.get(timeout=90)
            results[rank] = out
    finally:
        for p in procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
    return results


def test_followers_replay_the_leaders_calls_in_order():
    res = _run(3, fail=False)
    assert res[0][0] == "ok", res[0]
    lead_log = res[0][1]
    for r in (1, 2):
        kind, passes, log, errors = res[r]
        assert kind == "follower" and errors == [] and passes == 4           # two forwards, encoder slice, replay slice
        assert log == lead_log
    assert [m[0] for m in lead_log] == ["admit", "ensure", "set_rows", "engram", "forward", "engram_clear", "snapshot",
                                        "logits", "set_rows", "forward", "ced_enc", "ced_replay", "restore_prefix",
                                        "restore", "drop", "release"]


def test_a_failing_follower_leaves_and_the_leader_stops_launching():
    res = _run(2, fail=True)
    assert res[1][0] == "follower" and "site 201" in res[1][3][0], res[1]
    assert res[0][0] == "rank failure", res[0]
    assert res[0][1] == [1] and "forward failed" in res[0][2][1]
