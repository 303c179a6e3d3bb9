"""The serving scheduler on a CPU stand-in for the engine: real page allocator, prefix banks and scheduler loop, a pass
that only derives a token from its inputs.  Failures are injected on the host (a pass that raises, a pool too small)."""
import math
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


def test_a_prompt_that_shares_only_a_leading_part_reuses_host_pages_up_to_the_cut(cpu_sampler):
    """Demoted snapshots also serve prompts that diverge from them: the rows of the shared part minus one window come
    back from the host (whole pages below the cut, the cut page only up to the cut - out of a host page, or out of the
    snapshot's partly filled last page), the window before the cut is replayed, and only the pages read are budgeted."""
    eng = FakeEngine(slots=2, max_ctx=512, n_pages=10)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64, host_cache_bytes=4 << 20)
    cache, tier = eng.cache, be.host_tier
    W, P = eng.cfg.window, cache.page_tokens
    assert (W, P) == (32, 64)
    try:
        long_, short = [1000 + i for i in range(130)], [3000 + i for i in range(114)]     # 2 pages + 2; 1 page + 50
        stamps = {}
        for name, prompt in (("long", long_), ("short", short)):
            r = _req(prompt, max_tokens=3)
            be.submit(r)
            assert _run(be, [r])[0][1] == "length"
            _idle(be)
            (toks, snap, _), = [v for v in be.snapshots.values() if len(v[0]) == len(prompt)]
            for src, pr in cache.page_rows.items():
                for n, pg in enumerate(snap.pages):
                    rows = cache.comp[src][pg * pr:(pg + 1) * pr]
                    rows.copy_((torch.arange(pr).float()[:, None] + 100 * n + 1000 * src + 7).expand_as(rows))
                    cache.idx[src][pg * pr:(pg + 1) * pr] = -cache.comp[src][pg * pr:(pg + 1) * pr, :cache.idx[src].shape[1]]
                c, ix = snap.partial[src]
                c.copy_((torch.arange(c.shape[0]).float()[:, None] + 5000 + 1000 * src).expand_as(c))
                ix.copy_(-c[:, :ix.shape[1]])
                stamps[(name, src)] = ([cache.comp[src][pg * pr:(pg + 1) * pr].clone() for pg in snap.pages], c.clone())
        big = _req([7 + i for i in range(440)], max_tokens=60)           # page pressure: both snapshots are demoted
        be.submit(big)
        assert _run(be, [big])[0][1] == "length"
        _idle(be)
        assert be.totals["snapshots_demoted"] >= 2
        for sid in list(be.snapshots):                                   # nothing on the "device" can serve the prompts
            be._drop_snapshot(sid)
        for pool in list(cache.comp.values()) + list(cache.idx.values()):
            pool.zero_()
        restored0 = tier.stats()["restored"]

        def diverging(base, common, tag):
            prompt = base[:common] + [9000 + tag * 100 + i for i in range(30)]
            hits0, partial0, passes0 = be.totals["prompt_cache_hit_tokens"], be.totals["partial_prefix_hits"], eng.passes
            r = _req(prompt, max_tokens=2)
            be.submit(r)
            assert _run(be, [r])[0][1] == "length"
            _idle(be)
            cut = common // 2 * 2 - W
            assert be.totals["prompt_cache_hit_tokens"] - hits0 == cut
            assert be.totals["partial_prefix_hits"] - partial0 == 1
            # the prompt snapshot and the turn snapshot of the finished request share the restored pages
            snap = [v[1] for v in be.snapshots.values() if tuple(v[0][:len(prompt)]) == tuple(prompt)][0]
            return cut, snap, eng.passes - passes0

        # 1) the cut (78) falls into the long snapshot's second whole page: page 0 whole, 14 positions of page 1
        cut, snap, passes = diverging(long_, 110, 1)
        assert cut == 78 and be.totals["host_tier_hits"] == 1
        for src, pr in cache.page_rows.items():
            whole, _ = stamps[("long", src)]
            rows = (14 * pr + P - 1) // P
            p0, p1 = snap.pages[0], snap.pages[1]
            assert torch.equal(cache.comp[src][p0 * pr:(p0 + 1) * pr], whole[0])
            assert torch.equal(cache.idx[src][p0 * pr:(p0 + 1) * pr], -whole[0][:, :cache.idx[src].shape[1]])
            assert torch.equal(cache.comp[src][p1 * pr:p1 * pr + rows], whole[1][:rows])
            assert not cache.comp[src][p1 * pr + rows:(p1 + 1) * pr].any()            # nothing beyond the cut came along
        assert tier.stats()["restored"] - restored0 == 2 and tier.stats()["promoted_partial"] == 1
        assert passes >= 2                                               # replay of [78, 110) + the new tokens + decode
        # 2) the cut (80) falls into the short snapshot's partly filled last page: one host page + 16 kept positions
        restored1 = tier.stats()["restored"]
        cut, snap, _ = diverging(short, 112, 2)
        assert cut == 80 and be.totals["host_tier_hits"] == 2
        for src, pr in cache.page_rows.items():
            whole, part = stamps[("short", src)]
            rows = (16 * pr + P - 1) // P
            p0, p1 = snap.pages[0], snap.pages[1]
            assert torch.equal(cache.comp[src][p0 * pr:(p0 + 1) * pr], whole[0])
            assert torch.equal(cache.comp[src][p1 * pr:p1 * pr + rows], part[:rows])
            assert not cache.comp[src][p1 * pr + rows:(p1 + 1) * pr].any()
        assert tier.stats()["restored"] - restored1 == 1
        # 3) a shared part shorter than one window is not worth a restore
        hits0 = be.totals["host_tier_hits"]
        r = _req(long_[:30] + [8000 + i for i in range(20)], max_tokens=2)
        be.submit(r)
        assert _run(be, [r])[0][1] == "length"
        assert be.totals["host_tier_hits"] == hits0 and tier.hc.check() == 0
    finally:
        be.close()


class FakeVision:
    """Stand-in for the vision tower: one row per placeholder, counted."""

    def __init__(self, hidden):
        self.hidden, self.encodes = hidden, 0

    def encode(self, patches, grid):
        self.encodes += 1
        return torch.zeros(grid[0] * grid[1], self.hidden)


def _image(tag, rows=40):
    from ds41rt_b200.serving.images import PreparedImage
    import numpy as np
    return PreparedImage(patches=np.full((rows, 12), float(tag), dtype=np.float32), grid=(rows, 1), rows=rows,
                         identity=f"picture-{tag}")


def test_prompts_with_images_are_banked_under_the_identity_of_their_pictures(cpu_sampler):
    """Placeholder tokens look alike, so the banks compare image keys at their positions: the same picture under the
    same text is a cache hit (and is not encoded again when all of its rows were restored), another picture at the same
    place shares only the text before it, and a text prompt with the bare placeholder token matches neither."""
    from ds41rt_b200.serving.imagekeys import FIRST_IMAGE_KEY, ImageKeySpace
    eng = FakeEngine(slots=2, max_ctx=512)
    vis = FakeVision(eng.cfg.hidden)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64, vision=vis)
    IMG, W = 5, eng.cfg.window
    head, tail = [100 + i for i in range(50)], [300 + i for i in range(30)]

    def ask(image, extra=(), first=50, text_only=False):
        prompt = head + [IMG] * 40 + tail + list(extra)
        r = _req(prompt, max_tokens=3)
        if not text_only:
            r.images = [(image, list(range(first, first + 40)))]
        hits0, enc0 = be.totals["prompt_cache_hit_tokens"], vis.encodes
        be.submit(r)
        toks, status = _run(be, [r])[0]
        assert status == "length"
        _idle(be)
        return toks, be.totals["prompt_cache_hit_tokens"] - hits0, vis.encodes - enc0

    try:
        cat, dog = _image(1), _image(2)
        cold, hit, enc = ask(cat)
        assert hit == 0 and enc == 1 and be.stats()["image_keys"] == {"live": 1, "issued": 1, "forgotten": 0}
        # the stored keys carry the image key at the picture's positions and real tokens elsewhere
        key, = {v[0][50] for v in be.snapshots.values()}
        assert key >= FIRST_IMAGE_KEY and all(v[0][49] == 149 and v[0][90] == 300 for v in be.snapshots.values())
        # same picture, longer text: everything up to the end of the stored turn is reused, nothing is encoded
        again, hit, enc = ask(cat, extra=cold[:2] + [777, 778])
        assert hit == 120 + 2 and enc == 0 and be.totals["image_encodes_skipped"] == 1
        # another picture at the same place: only the text before it (minus one window, replayed) is shared
        other, hit, enc = ask(dog)
        assert hit == 50 // 2 * 2 - W and enc == 1 and be.totals["partial_prefix_hits"] == 1
        assert other == cold                                              # the stand-in engine ignores pixels
        # the same picture again after the other one: full hit on its own snapshot (logits included: no pass at all)
        same, hit, enc = ask(cat)
        assert same == cold and hit == 120 and enc == 0
        # the bare placeholder token in a text prompt is not an image: it shares the text before the picture only
        _, hit, enc = ask(None, text_only=True)
        assert hit == 50 // 2 * 2 - W and enc == 0
        assert be.stats()["image_keys"]["issued"] == 2
    finally:
        be.close()
    # the key space: keys are single-use, a forgotten picture comes back under a new key, bad spans are not keyed
    ks = ImageKeySpace(capacity=2)
    toks = [9] * 8
    k1 = ks.prepare(toks, [(_image(1), [0, 1])]).bindings[0][1]
    k2 = ks.prepare(toks, [(_image(2), [2, 3])]).bindings[0][1]
    assert ks.prepare(toks, [(_image(1), [4])]).bindings == [(4, k1)]
    ks.prepare(toks, [(_image(3), [5])])                                    # capacity 2: picture 2 is forgotten
    k2b = ks.prepare(toks, [(_image(2), [2])]).bindings[0][1]
    assert len({k1, k2, k2b}) == 3 and k2b > k2 and ks.stats()["forgotten"] >= 1
    both = ks.prepare(toks, [(_image(1), [0, 1]), (_image(1), [4, 5])])
    assert both.encode(toks)[:6] == [both.bindings[0][1]] * 2 + [9, 9] + [both.bindings[0][1]] * 2
    assert both.encode(toks[:1]) == [both.bindings[0][1]]
    assert ks.prepare(toks, [(_image(1), [7, 8])]) is None                  # outside the prompt
    assert ks.prepare(toks, [(_image(1), [0]), (_image(2), [0])]) is None   # one position, two pictures
    assert ks.prepare([9, 8], [(_image(1), [0, 1])]) is None                # different placeholder tokens
    ks.next = (1 << 32)
    assert ks.prepare(toks, [(_image(7), [0])]) is None                     # key range used up: not banked


class FakeSpec:
    """Stand-in for runtime.speculative.SpecSession over the CPU engine above: the "drafter" knows the engine's token
    rule and proposes the true continuation, except that every `wrong_every`-th proposed token is off by one."""

    def __init__(self, eng, width=5, wrong_every=3, confident=False):
        self.e, self.width, self.wrong_every, self.confident = eng, width, wrong_every, confident
        self.last_confidence = []
        self.proposed = 0
        self.calls = {"draft_groups": 0, "verify_groups": 0, "draft": 0, "verify": 0, "feed": 0}

        class _D:
            max_groups = 4

            def feed(_self, n):
                self.calls["feed"] += 1
        self.d = _D()

    @staticmethod
    def rule(tok, pos):
        return (tok * 31 + pos * 7 + 3) % 1000 + 2

    def _propose(self, anchor, pos):
        out, tok = [], anchor
        for j in range(self.width - 1):
            tok = self.rule(tok, pos + j)
            self.proposed += 1
            out.append(tok + 1 if self.proposed % self.wrong_every == 0 else tok)
            tok = out[-1]
        return out

    def draft_host_groups(self, slots, anchors, positions):
        self.calls["draft_groups"] += 1
        props = [self._propose(a, p) for a, p in zip(anchors, positions)]
        if not self.confident:
            return props, [[] for _ in slots]
        # a confidence head that knows: high where the proposal is the true continuation, low where it is off
        confs = []
        for a, p, prop in zip(anchors, positions, props):
            tok, c = a, []
            for j, t in enumerate(prop):
                c.append(0.95 if t == self.rule(tok, p + j) else 0.05)
                tok = t
            confs.append(c + [0.5])
        return props, confs

    def verify_host_groups(self, slots, inputs, positions):
        self.calls["verify_groups"] += 1
        toks, pos, first = [], [], []
        for inp, p in zip(inputs, positions):
            first.append(len(toks))
            toks += inp
            pos += list(range(p, p + len(inp)))
        self.e.set_rows(toks, pos, [0] * len(toks))
        self.e.forward_rows(len(toks))
        return first

    def draft_host(self, slot, anchor, pos):
        self.calls["draft"] += 1
        return self._propose(anchor, pos)

    def verify_host(self, slot, inputs, pos):
        self.calls["verify"] += 1
        self.e.set_rows(inputs, list(range(pos, pos + len(inputs))), [slot] * len(inputs))
        self.e.forward_rows(len(inputs))

    def prime(self, slot, anchor, pos):
        self.state = [slot, anchor, pos]

    def round_host(self):
        """The all-device round of a lone greedy request, done on the host here."""
        slot, anchor, pos = self.state
        drafts = self._propose(anchor, pos)
        self.verify_host(slot, [anchor] + drafts, pos)
        chosen = self.e.chosen[: len(drafts) + 1].tolist()
        k = 0
        while k < len(drafts) and chosen[k] == drafts[k]:
            k += 1
        self.state = [slot, chosen[k], pos + k + 1]
        return chosen[: k + 1]


def test_shared_speculative_rounds_emit_exactly_the_plain_tokens(cpu_sampler):
    """Scheduler side of the rounds that several requests share: proposals are cut at each request's budget, every
    request keeps the drafts that equal the verification rows' own tokens plus one more, a request that finishes
    inside a round leaves the others running - and everyone receives what plain decoding would have given."""
    from ds41rt_b200.runtime import core as K

    def expected(prompt, n):
        tok, pos, out = FakeSpec.rule(prompt[-1], len(prompt) - 1), len(prompt), []
        out.append(tok)
        while len(out) < n:
            tok = FakeSpec.rule(tok, pos)
            pos += 1
            out.append(tok)
        return out

    eng = FakeEngine(slots=4, max_rows=64)
    be = NativeBackend(eng, eos=1, concurrency=4, prefill_chunk=64, use_graphs=False)
    try:
        spec = FakeSpec(eng)
        be.policy, be.policy_lanes = K.DSparkPolicy(max_width=4), K.DSparkPolicy(max_width=4)
        be.spec_lanes = 4
        be.spec = spec                                     # from here on admitted requests are followed by the drafter
        prompts = [list(range(10, 50)), list(range(60, 93)), list(range(200, 247))]
        budgets = [23, 9, 16]
        reqs = [_req(p, n) for p, n in zip(prompts, budgets)]
        for r in reqs:
            be.submit(r)
        got = _run(be, reqs)
        for (toks, status), p, n in zip(got, prompts, budgets):
            assert status == "length" and toks == expected(p, n)
        assert be.healthy, be.error
        t = be.totals
        assert t["spec_lane_rounds"] > 0 and spec.calls["draft_groups"] == spec.calls["verify_groups"] > 0
        assert t["spec_tokens"] > t["spec_rounds"]          # drafts were accepted (two of three proposals are right)
        _idle(be)
    finally:
        be.close()


def test_shared_rounds_verify_fewer_rows_when_the_drafter_says_where_it_is_unsure(cpu_sampler):
    """With a confidence head the lengths of a shared round are chosen together from the per-position confidences:
    rows behind a draft the head doubts are not verified, the tokens stay exactly the plain ones, and a larger share of
    the verified drafts is kept than without the head."""
    from ds41rt_b200.runtime import core as K

    def serve(confident):
        eng = FakeEngine(slots=4, max_rows=64)
        be = NativeBackend(eng, eos=1, concurrency=4, prefill_chunk=64, use_graphs=False)
        try:
            spec = FakeSpec(eng, confident=confident)
            be.policy = K.DSparkPolicy(max_width=4)
            be.policy_lanes = pol = K.DSparkPolicy(max_width=4, warmup_rounds=4)
            # what a timed engine would have taught the policy (the CPU stand-in has no device clock): a request's
            # share of a round is dominated by its fixed part, a shared round costs 1000 + 300 us per row
            for w in (0, 1, 2, 3, 4, 4, 2):
                pol.observe(w, w, 1000.0 + 10.0 * (1 + w))
            for rows in (3, 6, 9, 12, 15):
                pol.observe_round(rows, 3, 1000.0 + 300.0 * rows)
            be.spec_lanes = 4
            be.spec = spec
            prompts = [list(range(10, 50)), list(range(60, 93)), list(range(200, 247))]
            reqs = [_req(p, 60) for p in prompts]
            for r in reqs:
                be.submit(r)
            got = _run(be, reqs)
            assert be.healthy, be.error
            _idle(be)
            return [g[0] for g in got], be.policy_lanes.stats(), dict(be.totals)
        finally:
            be.close()

    plain_toks, plain_stats, plain_totals = serve(False)
    toks, stats, totals = serve(True)
    assert toks == plain_toks and all(len(t) == 60 for t in toks)
    j = stats["joint"]
    assert j["draft_rows_offered"] > 0 and j["draft_rows_taken"] < j["draft_rows_offered"]
    assert plain_stats["joint"]["draft_rows_offered"] == 0            # no head: the joint choice is never asked
    assert totals["spec_lane_rounds"] > 0 and j["draft_rows_taken"] > 0
    # rows the head doubted were not verified: of the draft rows that were, a larger share was kept than with no head
    accepted = lambda st: sum(i * n for i, n in enumerate(st["accepted_histogram"]))
    assert (accepted(stats) - 16) / j["draft_rows_taken"] > 0.7      # 16: the accepted drafts of the taught rounds
    a, b = stats["joint"]["platt_positions"]
    assert 1 / (1 + math.exp(-(a * 0.95 + b))) > 1 / (1 + math.exp(-(a * 0.05 + b)))    # the calibration learnt the head


def test_prefill_matrix_tool_reports_cold_and_retained_rows(cpu_sampler):
    """utils.prefill_matrix over the CPU stand-in: a retained row restores the base from the snapshot an earlier request
    left and computes only what follows, a cold row computes everything."""
    from ds41rt_b200.utils.prefill_matrix import run_matrix
    eng = FakeEngine(slots=2, max_ctx=1024, max_rows=64)
    be = NativeBackend(eng, eos=1, concurrency=1, prefill_chunk=64)
    try:
        rows = run_matrix(be, eng.cfg.vocab, [0, 192], [32, 96], warm=False)
        assert be.healthy, be.error
    finally:
        be.close()
    assert [(r["base"], r["suffix"], r["mode"]) for r in rows] == [
        (0, 32, "cold"), (0, 96, "cold"), (192, 32, "cold"), (192, 32, "retained"), (192, 96, "cold"), (192, 96, "retained")]
    for r in rows:
        if r["mode"] == "cold":
            assert r["cache_hit_tokens"] == 0 and r["computed_tokens"] == r["base"] + r["suffix"]
        else:
            assert 0 < r["cache_hit_tokens"] <= r["base"] and r["computed_tokens"] < r["base"] + r["suffix"]


def test_a_request_cancelled_between_shared_rounds_leaves_the_others_exact(cpu_sampler):
    """Cancellation is looked at between rounds: the cancelled request retires, its slot and pages come back, and the
    requests that shared its speculative rounds still receive exactly the plain tokens."""
    from ds41rt_b200.runtime import core as K
    eng = FakeEngine(slots=4, max_rows=64)
    be = NativeBackend(eng, eos=1, concurrency=4, prefill_chunk=64, use_graphs=False)
    try:
        be.policy, be.policy_lanes = K.DSparkPolicy(max_width=4), K.DSparkPolicy(max_width=4)
        be.spec_lanes = 4
        be.spec = FakeSpec(eng, wrong_every=4)
        prompts = [list(range(10, 50)), list(range(60, 93)), list(range(200, 247))]
        reqs = [_req(prompts[0], 400), _req(prompts[1], 30), _req(prompts[2], 26)]
        for r in reqs:
            be.submit(r)
        # wait for the long request's first tokens, then cancel it
        first = reqs[0].events.get(timeout=10)
        while first.kind != "tokens":
            first = reqs[0].events.get(timeout=10)
        reqs[0].cancelled.set()
        got = _run(be, reqs[1:])
        for (toks, status), p, n in zip(got, prompts[1:], (30, 26)):
            tok, pos, want = FakeSpec.rule(p[-1], len(p) - 1), len(p), []
            want.append(tok)
            while len(want) < n:
                tok = FakeSpec.rule(tok, pos)
                pos += 1
                want.append(tok)
            assert status == "length" and toks == want
        tail = _run(be, [reqs[0]])[0]
        assert tail[1] == "cancelled" and be.healthy
        _idle(be)
        assert not be.active and eng.cache.free_pages == eng.cache.n_pages - sum(
            len(s[1].pages) for s in be.snapshots.values())
        assert be.totals["spec_lane_rounds"] > 0
    finally:
        be.close()


def test_probe_rounds_bring_speculation_back_when_drafts_become_right(cpu_sampler):
    """A policy that gave up on drafting answers every few decisions with a probe; the probe round keeps its width through
    the second, confidence-conditioned look, so its outcome is observed and speculation resumes once drafts are accepted."""
    from ds41rt_b200.runtime import core as K
    eng = FakeEngine(slots=2, max_rows=64)
    be = NativeBackend(eng, eos=1, concurrency=2, prefill_chunk=64, use_graphs=False)
    try:
        spec = FakeSpec(eng, wrong_every=1)               # every proposed token is wrong
        spec.last_confidence = [0.5] * spec.width         # a confidence head: the round asks the policy a second time
        be.policy, be.policy_lanes = K.DSparkPolicy(max_width=4, warmup_rounds=4), K.DSparkPolicy(max_width=4)
        be.policy.probe(8)
        for w in (4, 0, 2, 4, 0, 2):                      # the cost side of the model: 1000 us + 150 us per row (a CPU
            be.policy.observe(w, 0, 1000 + 150 * (1 + w), 20.0 * w)       # engine has no device clock to learn it from)
        be.spec = spec
        sampled = Sampling(temperature=0.7, seed=11)      # not the all-device round: drafts are read back and cut
        r = GenRequest(prompt_ids=list(range(10, 50)), max_tokens=120, sampling=sampled)
        be.submit(r)
        toks, status = _run(be, [r])[0]
        assert status == "length" and len(toks) == 120
        t1 = dict(be.totals)
        assert t1["policy_plain_rounds"] > 20 and be.policy.probe() >= 2      # it gave up, then probed
        verified_while_wrong = spec.calls["verify"]
        spec.wrong_every = 10 ** 9                        # from now on every draft is right
        _idle(be)
        be.snapshots.clear()
        r2 = GenRequest(prompt_ids=list(range(60, 100)), max_tokens=200, sampling=sampled)
        be.submit(r2)
        toks2, status2 = _run(be, [r2])[0]
        assert status2 == "length" and len(toks2) == 200
        t2 = be.totals
        # accepted probes switched speculation back on: far fewer rounds than tokens for the second request
        assert t2["spec_tokens"] - t1["spec_tokens"] > 100
        assert (t2["rounds"] - t1["rounds"]) < 150 and spec.calls["verify"] > verified_while_wrong
        assert be.policy.choose() > 0
    finally:
        be.close()


def test_a_request_that_does_not_fit_waits_for_a_retirement(cpu_sampler):
    """With requests active and the page pool short, a new request is parked, not refused: it is admitted when an
    earlier request retires and then runs to completion.  A cancelled parked request never starts."""
    eng = FakeEngine(slots=3, max_ctx=512, n_pages=7)        # 64-token pages: room for two of the requests below
    be = NativeBackend(eng, eos=1, concurrency=3, prefill_chunk=64, prompt_snapshots=0, turn_snapshots=0)
    try:
        a, b, c = _req(range(10, 150), 40), _req(range(200, 340), 40), _req(range(400, 540), 12)
        for r in (a, b, c):
            be.submit(r)
        d = _req(range(600, 740), 12)
        be.submit(d)
        d.cancelled.set()                                     # queued behind the parked one and cancelled before it starts
        got = _run(be, [a, b, c])
        assert [s for _, s in got] == ["length"] * 3 and [len(t) for t, _ in got] == [40, 40, 12]
        assert be.healthy and be.totals["failed"] == 0
        _idle(be)
        assert eng.cache.free_pages == eng.cache.n_pages and be.pending is None
        assert d.events.empty() or all(ev.kind != "tokens" for ev in list(d.events.queue))
    finally:
        be.close()


def test_stop_tokens_end_a_request_inside_a_shared_round_like_in_plain_decoding(cpu_sampler):
    """A stop token that the drafter proposed correctly must not be 'accepted and walked past': the request ends at it,
    in a shared speculative round exactly as in a plain step."""
    from ds41rt_b200.runtime import core as K

    def chain(prompt, n):
        tok, pos, out = FakeSpec.rule(prompt[-1], len(prompt) - 1), len(prompt), []
        out.append(tok)
        while len(out) < n:
            tok = FakeSpec.rule(tok, pos)
            pos += 1
            out.append(tok)
        return out

    prompts = [list(range(10, 50)), list(range(60, 93)), list(range(200, 247))]
    stops = [chain(prompts[0], 40)[6], chain(prompts[1], 40)[11], chain(prompts[2], 40)[1]]

    def run(with_spec):
        eng = FakeEngine(slots=4, max_rows=64)
        be = NativeBackend(eng, eos=1, concurrency=4, prefill_chunk=64, use_graphs=False)
        try:
            if with_spec:
                be.policy, be.policy_lanes = K.DSparkPolicy(max_width=4), K.DSparkPolicy(max_width=4)
                be.spec_lanes = 4
                be.spec = FakeSpec(eng, wrong_every=10 ** 9)          # every draft is right: stops sit inside accepted runs
            reqs = [GenRequest(prompt_ids=p, max_tokens=40, sampling=Sampling(), stop_ids=[s])
                    for p, s in zip(prompts, stops)]
            for r in reqs:
                be.submit(r)
            out = _run(be, reqs)
            assert be.healthy, be.error
            return out, dict(be.totals)
        finally:
            be.close()

    plain, _ = run(False)
    spec, totals = run(True)
    assert plain == spec and totals["spec_lane_rounds"] > 0
    for (toks, status), p, s in zip(spec, prompts, stops):
        want = chain(p, 40)
        cut = want.index(s)
        assert status == "stop" and toks == want[:cut]               # the stop token itself is not delivered
