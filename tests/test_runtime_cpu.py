"""Host runtime: admission, lanes, dSpark policy, host snapshot cache with a stub copy engine (no GPU)."""
import math
import random

import pytest

from ds41rt_b200.runtime import core as K


def test_admission_bounds_queue_and_waiters():
    a = K.Admission(queue_cap=2, waiter_cap=1)
    assert [a.reserve() for _ in range(4)] == [0, 0, 1, -1]
    a.release()                      # the waiter takes the freed place
    assert a.stats()["waiting"] == 0 and a.stats()["queued"] == 2
    assert a.reserve() == 1 and a.reserve() == -1
    assert a.stats()["rejected"] == 2


def test_lanes_balance_and_round_plan():
    l = K.Lanes(2)
    lanes = [l.add(i, remaining=10, history=500) for i in range(5)]
    assert lanes == [0, 1, 0, 1, 0] and l.load(0) == 3 and l.load(1) == 2
    l.retire(1)
    l.retire(3)                      # lane 1 empty -> one request moves over
    assert abs(l.load(0) - l.load(1)) <= 1
    l2 = K.Lanes(1)
    l2.add(10, remaining=100, history=500)
    l2.add(11, remaining=1, history=500)       # one token left: anchor only
    l2.add(12, remaining=100, history=3)       # short history: anchor only
    l2.add(13, remaining=3, history=500)       # never verify more rows than tokens remain
    assert l2.plan_round(0, draft_len=4, max_rows=64, min_history=16) == [(10, 5), (11, 1), (12, 1), (13, 3)]
    assert l2.plan_round(0, draft_len=4, max_rows=7, min_history=16) == [(10, 5), (11, 1), (12, 1)]


def test_joint_policy_spends_rows_where_they_are_likely_to_be_kept():
    """Lengths of a shared round are chosen together: the round costs A + B x rows, so rows go to the positions most
    likely to be committed, and the choice equals an exhaustive search over all length combinations."""
    import itertools
    rng = random.Random(1)
    pol = K.DSparkPolicy(max_width=4, warmup_rounds=8)
    assert pol.choose_joint([[0.9] * 4, [0.1] * 3]) == [4, 3]                   # warm-up: verify everything offered
    # world: a draft with confidence c is right with probability c (chains stop at the first wrong one);
    # a shared round of R rows takes 2000 + 400 R microseconds
    def play(confs, widths):
        out = []
        for c, w in zip(confs, widths):
            k = 0
            while k < w and rng.random() < c[k]:
                k += 1
            out.append(k)
        return out
    for _ in range(600):
        confs = [[rng.choice([0.15, 0.5, 0.95])] * 4 for _ in range(rng.randint(2, 4))]
        widths = [rng.randint(0, 4) for _ in confs]
        rows = sum(1 + w for w in widths)
        for c, w, k in zip(confs, widths, play(confs, widths)):
            pol.observe(w, k, -1.0, confidence=c[0] if w else -1.0)
            pol.observe_positions(c, w, k)
        pol.observe_round(rows, len(confs), 2000.0 + 400.0 * rows)
    st = pol.stats()["joint"]
    assert abs(st["round_fixed_us"] - 2000.0) < 1.0 and abs(st["round_us_per_row"] - 400.0) < 0.5 and st["rounds"] == 600
    # calibration: the fitted curve orders and roughly places the three confidence levels
    a, b = st["platt_positions"]
    cal = lambda c: 1.0 / (1.0 + math.exp(-(a * c + b)))
    assert cal(0.15) < 0.35 and 0.3 < cal(0.5) < 0.7 and cal(0.95) > 0.8
    sure, unsure = [0.95] * 4, [0.15] * 4
    got = pol.choose_joint([sure, unsure, [0.5] * 4])
    assert got[0] >= 3 and got[1] == 0 and got[0] >= got[2] >= got[1]
    # the same objective by brute force, with the policy's own probabilities
    def prob(c, depth):
        return 0.5 * pol.acceptance(depth) + 0.5 * cal(c)
    def value(confs, widths):
        tokens = sum(1 + sum(math.prod(prob(c[j], j + 1) for j in range(k + 1)) for k in range(w))
                     for c, w in zip(confs, widths))
        return tokens / (st["round_fixed_us"] + st["round_us_per_row"] * sum(1 + w for w in widths))
    for confs in ([sure, unsure, [0.5] * 4], [[0.95, 0.5, 0.5, 0.15], [0.5, 0.95, 0.95, 0.95]], [unsure, unsure]):
        best = max(itertools.product(range(5), repeat=len(confs)), key=lambda ws: value(confs, ws))
        got = pol.choose_joint(confs)
        assert value(confs, got) >= value(confs, best) * (1 - 1e-6), (confs, got, best)
    # a chain is only as good as its weakest earlier link: sure drafts behind an unlikely one count for little
    weak_first, strong = pol.choose_joint([[0.05, 0.99, 0.99, 0.99], [0.95] * 4] * 2)[:2]
    assert weak_first < strong
    # expensive rows (a pass dominated by per-row work) make the policy stingy, cheap rows generous
    dear, cheap = K.DSparkPolicy(max_width=4, warmup_rounds=0), K.DSparkPolicy(max_width=4, warmup_rounds=0)
    for rows in (2, 4, 6, 8, 10):
        dear.observe_round(rows, 2, 10.0 + 1000.0 * rows)
        cheap.observe_round(rows, 2, 5000.0 + 1.0 * rows)
    mid = [[0.6] * 4, [0.6] * 4]
    assert sum(cheap.choose_joint(mid)) == 8 and sum(dear.choose_joint(mid)) < 8
    assert pol.stats()["joint"]["draft_rows_taken"] <= pol.stats()["joint"]["draft_rows_offered"]
    assert pol.choose_joint([]) == [] and pol.choose_joint([[]]) == [0]


def test_policy_matches_exhaustive_search_after_warmup():
    rng = random.Random(0)
    pol = K.DSparkPolicy(max_width=4, warmup_rounds=12)
    assert pol.choose() == 4
    # environment: acceptance 0.9 per depth, pass time 1000 us + 150 us per row, drafting 20 us per row
    acc = 0.9
    for _ in range(400):
        w = rng.randint(0, 4)
        n = 0
        while n < w and rng.random() < acc:
            n += 1
        pol.observe(w, n, 1000 + 150 * (1 + w), 20.0 * w)
    best, best_w = -1, 0
    for w in range(5):
        benefit = 1 + sum(acc ** j for j in range(1, w + 1))
        cost = 1000 + 150 * (1 + w) + 20 * w
        if benefit / cost > best:
            best, best_w = benefit / cost, w
    assert pol.choose() == best_w == 4
    assert abs(pol.acceptance(1) - acc) < 0.1
    # hopeless drafts: stop verifying them
    bad = K.DSparkPolicy(max_width=4, warmup_rounds=4)
    for _ in range(100):
        bad.observe(4, 0, 1000 + 150 * 5, 80.0)
        bad.observe(0, 0, 1000 + 150, 0.0)
    assert bad.choose() == 0
    # ... but keep probing: every 8th plain decision is a two-draft probe, and once the probes are accepted the policy
    # returns to speculation
    bad.probe(8)
    picks = [bad.choose() for _ in range(16)]
    assert picks.count(2) == 2 and picks.count(0) == 14 and picks[6] == 2 and bad.probe() == 2
    for _ in range(200):
        w = bad.choose()
        if w > 0:
            bad.observe(w, w, 1000 + 150 * (1 + w), 20.0 * w)       # the text became predictable
    assert bad.choose() == 4
    bad.probe(0)                                                    # probing can be switched off
    never = K.DSparkPolicy(max_width=4, warmup_rounds=2)
    never.probe(0)
    for _ in range(50):
        never.observe(4, 0, 1750, 80.0)
        never.observe(0, 0, 1150, 0.0)
    assert [never.choose() for _ in range(200)].count(0) == 200
    s = pol.stats()
    assert s["rounds"] == 400 and abs(s["t_row_us"] - 150) < 5 and abs(s["t_fixed_us"] - 1000) < 20


def test_hostcache_sharing_budgets_eviction_and_failure():
    hc = K.HostCache(n_pages=8, page_bytes=1000, store_budget=5000, restore_budget=3000)
    r, pages, need = hc.store(1, [11, 12, 13], tokens=192)
    assert r == 3 and need == [True, True, True]
    r, pages2, need2 = hc.store(2, [11, 12, 99])            # shares two pages exactly, uses the remaining budget
    assert r == 3 and need2 == [False, False, True] and pages2[:2] == pages[:2]
    assert hc.store(3, [21, 22, 23])[0] == 0                # store budget exhausted this tick -> deferred
    hc.tick()
    assert hc.store(3, [21, 22, 23])[0] == 3
    assert hc.restore(1)[0] == 3
    assert hc.restore(2)[0] == 0                            # restore budget (3000) used up
    hc.tick()
    assert hc.restore(2)[0] == 3 and hc.restore(42)[0] == -1
    # pool has 8 pages, 7 in use: a 3-page snapshot forces eviction of the least recently used one (id 3)
    assert hc.store(4, [31, 32, 33])[0] == 3
    assert not hc.contains(3) and hc.contains(1) and hc.contains(2)
    assert hc.check() == 0
    # failed copy: the store is rolled back and leaves no pages behind
    eng = K.StubCopyEngine(latency_us=5, gb_per_s=10)
    eng.fail_at(1)
    hc.tick()
    r, pages, need = hc.store(5, [41, 42])
    ok = all(eng.copy(1000) >= 0 for n in need if n)
    assert not ok
    hc.abort(5)
    assert not hc.contains(5) and hc.check() == 0 and hc.metrics()["failed"] == 1
    assert eng.now_us > 0


def test_hostcache_randomised_simulation_keeps_invariants():
    rng = random.Random(7)
    hc = K.HostCache(n_pages=32, page_bytes=4096, store_budget=20 * 4096, restore_budget=20 * 4096)
    eng = K.StubCopyEngine()
    live = set()
    for step in range(2000):
        op = rng.random()
        sid = rng.randint(0, 40)
        if op < 0.5:
            keys = [rng.randint(0, 60) for _ in range(rng.randint(1, 6))]
            keys = list(dict.fromkeys(keys))
            r, pages, need = hc.store(sid, keys)
            if r > 0:
                if rng.random() < 0.05:
                    hc.abort(sid)
                    live.discard(sid)
                else:
                    for n in need:
                        if n:
                            eng.copy(4096)
                    live.add(sid)
        elif op < 0.8:
            r, pages = hc.restore(sid)
            assert (r >= 0) == hc.contains(sid)
        elif op < 0.9:
            hc.drop(sid)
        else:
            hc.tick()
        assert hc.check() == 0, step
    m = hc.metrics()
    assert m["evictions"] > 0 and m["shared"] > 0 and m["hits"] > 0


def test_trace_targets_follow_the_env_filter(monkeypatch):
    import importlib
    import logging
    from ds41rt_b200.utils import trace
    monkeypatch.setenv("DS41_LOG", "timing,sampling=debug")
    importlib.reload(trace)
    assert trace.enabled("timing") and not trace.enabled("timing", logging.DEBUG)
    assert trace.enabled("sampling", logging.DEBUG)
    assert not trace.enabled("host_cache")
    monkeypatch.delenv("DS41_LOG")
    importlib.reload(trace)
    assert not trace.enabled("timing")
