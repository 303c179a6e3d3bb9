"""The serving scheduler on a CPU stand-in for the engine: real page allocator, prefix banks and scheduler loop, a pass
that only derives a token from its inputs.  Failures are injected on the host (a pass that raises, a pool too small)."""
import queue
import time

import pytest
import torch

from ds41rt_b200.config import ModelConfig
from ds41rt_b200.models.ds41 import KVCache
from ds41rt_b200.serving.engine import GenRequest, NativeBackend
from ds41rt_b200.serving.protocol import Sampling


class FakeEngine:
    def __init__(self, slots=2, max_ctx=512, n_pages=None, max_rows=64):
        self.cfg = ModelConfig.tiny()
        self.device = torch.device("cpu")
        self.max_rows = max_rows
        self.cache = KVCache(self.cfg, self.cfg.n_layers, slots, max_ctx, self.device, n_pages=n_pages)
        self.chosen = torch.zeros(max_rows, dtype=torch.int32)
        self.last_head_row = 0
        self.fail_passes = 0
        self.passes = 0
        self.image_patch = None

    def set_rows(self, tokens, positions, slots, row_lo=None):
        self._rows = (list(tokens), list(positions))

    def forward_rows(self, rows, head=True, sources=True, **kw):
        if self.fail_passes:
            self.fail_passes -= 1
            raise RuntimeError("injected pass failure")
        self.passes += 1
        toks, pos = self._rows
        for i in range(rows):
            self.chosen[i] = (toks[i] * 31 + pos[i] * 7 + 3) % 1000 + 2
        self.last_head_row = rows - 1

    def logits_rows(self, rows):
        out = torch.zeros(rows, self.cfg.vocab)
        for i in range(rows):
            out[i, int(self.chosen[i])] = 10.0
        return out

    def ced_usable(self, start, n):
        return False

    def check_status(self, what=""):
        pass


@pytest.fixture
def cpu_sampler(monkeypatch):
    import ds41rt_b200.ops.sampling as S
    monkeypatch.setattr(S, "pack_params", lambda params, device: params)
    monkeypatch.setattr(S, "sample_rows", lambda logits, params, arena=None: (logits.argmax(-1).int(),
                                                                              torch.zeros(len(params), dtype=torch.int32)))


def _run(backend, reqs, timeout=20.0):
    out = []
    for r in reqs:
        toks, status, done, deadline = [], None, False, time.time() + timeout
        while not done and time.time() < deadline:
            try:
                ev = r.events.get(timeout=0.2)
            except queue.Empty:
                continue
            if ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                status, done = ev.reason, True
            elif ev.kind == "error":
                status, done = ("error", ev.status, ev.message), True
        out.append((toks, status))
    return out


def _idle(backend, timeout=5.0):
    """The finish event leaves before the slot is released: wait for the worker to be done with its requests."""
    deadline = time.time() + timeout
    while time.time() < deadline and (backend.active or backend.prefilling is not None or not backend.q.empty()):
        time.sleep(0.01)
    time.sleep(0.05)


def _req(prompt, max_tokens=4):
    return GenRequest(prompt_ids=list(prompt), max_tokens=max_tokens, sampling=Sampling())


def test_a_failed_prompt_pass_fails_only_its_request(cpu_sampler):
    eng = FakeEngine()
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64)
    try:
        eng.fail_passes = 1
        bad, good = _req(range(10, 50)), _req(range(60, 100))
        be.submit(bad)
        be.submit(good)
        (t0, s0), (t1, s1) = _run(be, [bad, good])
        assert s0[0] == "error" and s0[1] == 500 and "prompt pass failed" in s0[2]
        assert s1 == "length" and len(t1) == 4
        assert be.healthy and be.totals["failed"] == 1
        _idle(be)
        assert eng.cache.free_pages == eng.cache.n_pages - sum(len(s[1].pages) for s in be.snapshots.values())
        # the failed request's slot is usable again
        again = _req(range(10, 50))
        be.submit(again)
        assert _run(be, [again])[0][1] == "length"
    finally:
        be.close()


def test_requests_near_the_context_limit_are_refused_at_admission(cpu_sampler):
    eng = FakeEngine(max_ctx=256)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64)
    try:
        r = _req(range(2, 200), max_tokens=56)         # 198 + 56 + 1 slack = 255 <= 256: fits
        be.submit(r)
        assert _run(be, [r])[0][1] == "length"
        r2 = _req(range(2, 200), max_tokens=58)        # 257 > 256
        be.submit(r2)
        st = _run(be, [r2])[0][1]
        assert st[0] == "error" and st[1] == 400
    finally:
        be.close()


def test_snapshots_give_way_when_the_page_pool_runs_short(cpu_sampler):
    # 2 slots x 8 pages of context, pool of 10 pages: snapshots of earlier prompts must be evicted for a full-context one
    eng = FakeEngine(slots=2, max_ctx=512, n_pages=10)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64)
    try:
        for k in range(4):                              # four distinct 130-token prompts: 2 full pages pinned each
            r = _req([1000 + 131 * k + i for i in range(130)], max_tokens=3)
            be.submit(r)
            assert _run(be, [r])[0][1] == "length"
        pinned = sum(len(s[1].pages) for s in be.snapshots.values())
        assert pinned >= 4
        big = _req([7 + i for i in range(440)], max_tokens=60)       # 440 + 60 + 1 = 501 tokens -> 8 pages
        be.submit(big)
        toks, st = _run(be, [big])[0]
        assert st == "length" and len(toks) == 60
        assert be.totals["snapshots_evicted_for_pages"] >= 1
    finally:
        be.close()


def test_prefix_banks_drive_reuse_and_decode_interleaves_with_prompt_passes(cpu_sampler):
    eng = FakeEngine(slots=2, max_ctx=1024, max_rows=64)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64)
    try:
        base = [5 + (i * 17) % 900 for i in range(300)]
        a = _req(base, max_tokens=3)
        be.submit(a)
        assert _run(be, [a])[0][1] == "length"
        hits0 = be.totals["prompt_cache_hit_tokens"]
        b = _req(base + [77, 78, 79], max_tokens=3)              # extends the stored prompt
        be.submit(b)
        assert _run(be, [b])[0][1] == "length"
        assert be.totals["prompt_cache_hit_tokens"] - hits0 == 300
        # a long prompt arrives while another request decodes: its passes alternate with decode rounds
        long_dec = _req([3, 4, 5, 6], max_tokens=40)
        be.submit(long_dec)
        time.sleep(0.05)
        rounds_before = be.totals["rounds"]
        newcomer = _req([9 + (i * 13) % 800 for i in range(64 * 6)], max_tokens=2)
        be.submit(newcomer)
        res = _run(be, [long_dec, newcomer])
        assert res[0][1] == "length" and res[1][1] == "length"
        assert be.totals["prefill_passes"] >= 6 and be.totals["rounds"] > rounds_before
        # cancellation is honoured between prompt passes
        c = _req([11 + (i * 7) % 700 for i in range(64 * 8)], max_tokens=2)
        c.cancelled.set()
        be.submit(c)
        _idle(be)
        st = be.stats()
        assert st["kv"]["prompt_bank"] >= 1 and st["active"] == 0
    finally:
        be.close()


def test_demoted_snapshots_come_back_from_the_host_tier(cpu_sampler):
    """A snapshot pushed out of the device banks by page pressure is copied into host pages; a prompt that extends it
    gets fresh device pages filled from them (rows, rings and carry intact) and counts its tokens as cache hits; two
    snapshots with a common first page share that host page."""
    eng = FakeEngine(slots=2, max_ctx=512, n_pages=10)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64, host_cache_bytes=4 << 20)
    cache, tier = eng.cache, be.host_tier
    try:
        first = [1000 + i for i in range(130)]                       # 2 full pages + 2 tokens
        r = _req(first, max_tokens=3)
        be.submit(r)
        assert _run(be, [r])[0][1] == "length"
        _idle(be)
        (sid, (toks, snap, _)), = [(k, v) for k, v in be.snapshots.items() if len(v[0]) == 130]
        stamp = {}
        for n, pg in enumerate(snap.pages):                          # recognisable rows in the snapshot's pages
            for src, pr in cache.page_rows.items():
                cache.comp[src][pg * pr:(pg + 1) * pr] = 0.5 + n + 10 * src
                cache.idx[src][pg * pr:(pg + 1) * pr] = -1.5 - n - 10 * src
                stamp[(n, src)] = (cache.comp[src][pg * pr].clone(), cache.idx[src][pg * pr].clone())
        snap.rings.fill_(3.25)
        sibling = first[:64] + [5000 + i for i in range(66)]          # same first page, different second page
        r = _req(sibling, max_tokens=3)
        be.submit(r)
        assert _run(be, [r])[0][1] == "length"
        big = _req([7 + i for i in range(440)], max_tokens=60)       # needs 8 of the 10 pages: the snapshots must go
        be.submit(big)
        assert _run(be, [big])[0][1] == "length"
        _idle(be)
        assert be.totals["snapshots_demoted"] >= 2 and sid not in be.snapshots
        m = tier.stats()
        assert m["shared"] >= 1 and m["entries"] >= 2                # the common first page is stored once
        for pool in list(cache.comp.values()) + list(cache.idx.values()):
            pool.zero_()                                             # nothing of the old rows is left on the "device"
        hits0 = be.totals["prompt_cache_hit_tokens"]
        again = _req(first + [77, 78, 79], max_tokens=2)
        be.submit(again)
        # look at the slot while the request is still active: restore happened at admission
        assert _run(be, [again])[0][1] == "length"
        assert be.totals["host_tier_hits"] == 1 and be.totals["prompt_cache_hit_tokens"] - hits0 == 130
        assert tier.stats()["promoted_tokens"] == 130
        # the turn snapshot of the finished request shares the restored pages: its first two pages carry the stamps
        ent = [v for v in be.snapshots.values() if tuple(v[0][:130]) == tuple(first)]
        assert ent
        pages = ent[0][1].pages
        for n in range(2):
            for src, pr in cache.page_rows.items():
                assert torch.equal(cache.comp[src][pages[n] * pr], stamp[(n, src)][0])
                assert torch.equal(cache.idx[src][pages[n] * pr], stamp[(n, src)][1])
        assert "host_cache" in be.stats()
    finally:
        be.close()
