"""Rank failure detection on the host: fake clock on an in-process store, and real gloo ranks where one leaves with
a note or goes silent.  No GPU is involved; a peer learns of the loss from the store before its next collective, or -
if that collective was already posted - from the collective's error, and then names the rank from the store."""
import multiprocessing as mp
import os
import time

import pytest

from ds41rt_b200.parallel.health import DictStore, Heartbeat, RankFailure


def test_silent_left_and_missing_ranks_with_a_fake_clock():
    now = [100.0]
    store = DictStore()
    hb = [Heartbeat(store, r, 4, max_age=2.0, clock=lambda: now[0], join_grace=1.0) for r in range(3)]   # rank 3 never joins
    assert hb[0].peers_down() == {}                  # still within the joining grace
    now[0] += 1.0
    assert hb[0].peers_down() == {3: "never joined"}
    now[0] += 0.5
    hb[0].beat(); hb[1].beat()                       # rank 2 goes silent
    now[0] += 1.0
    down = hb[0].peers_down()
    assert set(down) == {2, 3} and down[2].startswith("silent")
    hb[1].leave("cuda status 2 at site 110")
    with pytest.raises(RankFailure) as e:
        hb[0].guard()
    assert e.value.ranks == [1, 2, 3] and "site 110" in e.value.reasons[1]


def _free_port_below_ephemeral():
    """A free port outside the range the kernel hands to outgoing connections: a client that retries against a port
    nobody listens on yet can otherwise be given that very port as its source and connect to itself."""
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


def test_an_unreachable_store_reports_every_peer():
    class Broken(DictStore):
        def check(self, keys):
            raise ConnectionError("Broken pipe")
    store = Broken()
    hb = Heartbeat(store, 0, 3)
    down = hb.peers_down()
    assert set(down) == {1, 2} and all(v.startswith("store unreachable") for v in down.values())
    with pytest.raises(RankFailure):
        hb.guard()


def _rank(rank, world, port, store_port, mode, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=False)      # hosted by the launcher
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=20))
    import torch
    hb = Heartbeat(store, rank, world, interval=0.05, max_age=1.5).start()
    hb.wait_joined(30.0)                             # ranks leave the rendezvous at slightly different times
    steps, failure = 0, None
    try:
        for step in range(60):
            hb.guard()                               # between steps: nothing in flight
            if rank == world - 1 and step == 3:
                if mode == "leave":
                    hb.leave("leaving after step 3")
                    break
                if mode == "die":
                    hb.stop()                        # goes silent without a note; stays out of further collectives
                    time.sleep(4.0)
                    break
            t = torch.ones(4)
            try:
                dist.all_reduce(t)
            except RuntimeError:
                # the peer left while this collective was already posted: the store says who and why
                deadline = time.time() + 5.0
                while time.time() < deadline and not hb.peers_down():
                    time.sleep(0.05)
                hb.guard()
                raise
            steps += 1
            time.sleep(0.05)
    except RankFailure as e:
        failure = (e.ranks, dict(e.reasons))
    except Exception as e:                           # anything else is reported, not left to hang the parent
        failure = ([], {"error": f"{type(e).__name__}: {e}"})
    q.put((rank, steps, failure))
    hb.stop()
    time.sleep(0.3)
    os._exit(0)                                      # no collective teardown with a missing peer


@pytest.mark.parametrize("mode", ["leave", "die"])
def test_gloo_ranks_detect_a_lost_peer_before_the_next_collective(mode):
    import torch.distributed as dist
    world = 3
    port = _free_port_below_ephemeral()
    # the heartbeat store lives in the launcher: it listens before any rank starts and outlives all of them
    host = dist.TCPStore("127.0.0.1", 0, None, is_master=True, wait_for_workers=False)
    store_port = host.port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, port, store_port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, steps, failure = q.get(timeout=60)
        results[rank] = (steps, failure)
    for p in procs:
        p.join(timeout=20)
    lost = world - 1
    assert results[lost][0] == 3
    for r in range(world - 1):
        steps, failure = results[r]
        assert failure is not None and lost in failure[0], results
        assert steps >= 3
        if mode == "leave":
            assert "leaving after step 3" in failure[1][lost]
        else:
            assert failure[1][lost].startswith("silent")
