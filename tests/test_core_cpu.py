"""Host runtime (C++ core) unit tests: sampler oracle, verification rule, Engram hashing, prefix banks, KV leases."""
import numpy as np
import pytest

from ds41rt_b200.runtime import core as K


# ---------------------------------------------------------------------------------------------- sampler
def test_greedy_lowest_id_tie_and_mask():
    logits = np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32)
    assert K.sample_token(logits) == 1
    mask = np.array([0b1101], dtype=np.uint32)        # token 1 disallowed
    assert K.sample_token(logits, mask) == 2
    assert K.sample_token(logits, temperature=0.7, top_k=1) == 1


def test_greedy_rejects_nonfinite_rows_and_empty_masks():
    with pytest.raises(K.SamplingError, match="nonfinite"):
        K.sample_token(np.array([0.0, np.nan], dtype=np.float32))
    with pytest.raises(K.SamplingError, match="empty"):
        K.sample_token(np.zeros(40, dtype=np.float32), np.zeros(2, dtype=np.uint32))
    with pytest.raises(K.SamplingError, match="mask_width"):
        K.sample_token(np.zeros(40, dtype=np.float32), np.zeros(3, dtype=np.uint32))
    with pytest.raises(K.SamplingError, match="invalid_temperature"):
        K.sample_token(np.zeros(4, dtype=np.float32), temperature=-1.0)


def test_categorical_follows_cdf_in_token_order():
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float32))
    picks = [K.sample_token(logits, temperature=1.0, uniform=u) for u in (0.05, 0.15, 0.45, 0.95)]
    assert picks == [0, 1, 2, 3]


def test_top_k_top_p_min_p_filters():
    logits = np.log(np.array([0.5, 0.25, 0.15, 0.10], dtype=np.float32))
    # top_k 2 renormalises over {0,1}: cdf 2/3, 1
    assert K.sample_token(logits, temperature=1.0, top_k=2, uniform=0.6) == 0
    assert K.sample_token(logits, temperature=1.0, top_k=2, uniform=0.7) == 1
    # top_p 0.7: nucleus {0,1} with mass 0.75; target = u * 0.75
    assert K.sample_token(logits, temperature=1.0, top_p=0.7, uniform=0.99) == 1
    # min_p 0.4: only tokens with p >= 0.4 * pmax = 0.2 survive -> {0,1}
    assert K.sample_token(logits, temperature=1.0, min_p=0.4, uniform=0.999) == 1


def test_distribution_matches_softmax_statistically():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=16).astype(np.float32)
    p = np.exp(logits / 0.8)
    p /= p.sum()
    counts = np.zeros(16)
    for i in range(4000):
        counts[K.sample_token(logits, temperature=0.8, uniform=K.sample_uniform(1234, i))] += 1
    assert np.abs(counts / 4000 - p).max() < 0.03


def test_uniform_depends_only_on_seed_and_position():
    a = [K.sample_uniform(7, i) for i in range(8)]
    assert a == [K.sample_uniform(7, i) for i in range(8)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) == 8
    assert K.sample_uniform(8, 0) != a[0]


def _sample_statement(logits, mask, temperature, top_k, top_p, min_p, u):
    """The sampling contract written out with numpy, independently of the library: masked softmax at the temperature,
    min_p against the best candidate, top-k (ties to the lower id), nucleus over what is left, inverse CDF at u."""
    n = len(logits)
    ok = np.ones(n, bool) if mask is None else np.array([(int(mask[i // 32]) >> (i % 32)) & 1 for i in range(n)], bool)
    if temperature < 1e-5 or top_k == 1:
        cand = np.where(ok)[0]
        return int(cand[np.argmax(logits[cand])])                   # argmax returns the first (lowest id) maximum
    scaled = (logits * np.float32(1.0 / np.float32(temperature))).astype(np.float32)
    top = scaled[ok].max()
    if min_p > 0:
        ok = ok & (scaled >= np.float32(top + np.float32(np.log(np.float32(min_p)))))
    cand = np.where(ok)[0]
    u = min(max(float(np.float32(u)), 0.0), 0.99999994)
    if top_k <= 0 and top_p >= 1.0:
        w = np.exp((scaled[cand] - top).astype(np.float64))          # token order
        run = np.cumsum(w)
        hit = np.where((run >= u * run[-1]) & (run > 0))[0]
        return int(cand[hit[0]]) if len(hit) else int(cand[-1])
    order = sorted(cand, key=lambda i: (-scaled[i], i))
    if 0 < top_k < len(order):
        order = order[:top_k]
    w = np.exp((scaled[order] - top).astype(np.float64))
    run = np.cumsum(w)
    keep, mass = len(order), run[-1]
    if top_p < 1.0:
        keep = int(np.where(run >= float(np.float32(top_p)) * run[-1])[0][0]) + 1
        mass = run[keep - 1]
    hit = np.where(run[:keep] >= u * mass)[0]
    return int(order[hit[0]]) if len(hit) else int(order[keep - 1])


def test_sampler_agrees_with_an_independent_statement_on_a_random_and_adversarial_corpus():
    rng = np.random.default_rng(5)
    checked = 0
    for case in range(600):
        n = int(rng.choice([3, 31, 32, 33, 64, 257, 300, 1000]))
        kind = case % 6
        logits = rng.normal(scale=3.0, size=n).astype(np.float32)
        if kind == 1:                                    # many exact ties, also at the top-k cut
            logits = rng.integers(-2, 3, size=n).astype(np.float32)
        elif kind == 2:                                  # a flat row: every weight equal
            logits[:] = 0.25
        elif kind == 3:                                  # huge spread: most weights underflow to subnormals or zero
            logits = (rng.normal(size=n) * 60).astype(np.float32)
        elif kind == 4:                                  # masked-out entries may be -inf
            logits[rng.random(n) < 0.2] = -np.inf
        mask = None
        if kind in (4, 5) or rng.random() < 0.3:
            bits = rng.random(n) < 0.6
            if kind == 4:
                bits &= np.isfinite(logits)
            if not bits.any():
                bits[int(np.argmax(np.where(np.isfinite(logits), logits, -1e30)))] = True
            mask = np.zeros((n + 31) // 32, dtype=np.uint32)
            for i in np.where(bits)[0]:
                mask[i // 32] |= np.uint32(1 << (i % 32))
        elif kind == 4:
            logits[~np.isfinite(logits)] = -50.0
        temperature = float(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5]))
        top_k = int(rng.choice([0, 1, 2, 5, 40, 256, 257, 500]))
        top_p = float(rng.choice([1.0, 0.95, 0.5, 0.1, 1e-6]))
        min_p = float(rng.choice([0.0, 0.05, 0.5, 1.0]))
        u = float(rng.choice([0.0, rng.random(), rng.random(), 0.9999999, 1.0]))
        if kind == 4 and (temperature < 1e-5 or top_k == 1):
            continue                                     # the greedy path wants a finite row even under the mask
        got = K.sample_token(logits, mask, temperature, top_k, top_p, min_p, u)
        want = _sample_statement(logits, mask, temperature, top_k, top_p, min_p, u)
        assert got == want, (case, n, temperature, top_k, top_p, min_p, u)
        if mask is not None:
            assert (int(mask[got // 32]) >> (got % 32)) & 1
        checked += 1
    assert checked > 500
    # the corners by hand: a tie at the top-k cut keeps the lower id; a nucleus of tiny top_p is the single best token;
    # min_p = 1 keeps only the best (and its exact ties); u = 1 is clamped into the last surviving token
    tie = np.array([1.0, 2.0, 2.0, 2.0, 0.0], dtype=np.float32)
    assert {K.sample_token(tie, temperature=1.0, top_k=2, uniform=u) for u in (0.0, 0.3, 0.6, 0.99)} == {1, 2}
    assert K.sample_token(tie, temperature=1.0, top_p=1e-6, uniform=0.999) == 1
    assert {K.sample_token(tie, temperature=1.0, min_p=1.0, uniform=u) for u in (0.0, 0.5, 0.99)} == {1, 2, 3}
    assert K.sample_token(tie, temperature=1.0, uniform=1.0) == 4
    # everything masked, +inf and NaN among the allowed entries are errors, never a token
    with pytest.raises(K.SamplingError, match="empty"):
        K.sample_token(tie, np.zeros(1, dtype=np.uint32), temperature=1.0, uniform=0.5)
    with pytest.raises(K.SamplingError, match="nonfinite"):
        K.sample_token(np.array([0.0, np.inf], dtype=np.float32), temperature=1.0, uniform=0.5)
    with pytest.raises(K.SamplingError, match="empty"):
        K.sample_token(np.array([-np.inf, -np.inf], dtype=np.float32), temperature=1.0, uniform=0.5)


# ---------------------------------------------------------------------------------------------- verification
def test_verify_accept_prefix():
    r = K.verify_greedy([10, 11, 12, 13], [11, 12, 99, 14], eos=1, remaining=100)
    assert r["emitted"] == [11, 12, 99] and r["accepted_inputs"] == 3 and not r["eos"]
    r = K.verify_greedy([10, 11], [50, 51], eos=1, remaining=100)
    assert r["emitted"] == [50] and r["accepted_inputs"] == 1
    r = K.verify_greedy([10, 11, 12], [11, 12, 13], eos=1, remaining=100)       # all accepted + bonus
    assert r["emitted"] == [11, 12, 13] and r["accepted_inputs"] == 3


def test_verify_stops_at_eos_and_length():
    r = K.verify_greedy([10, 1, 12], [1, 12, 13], eos=1, remaining=100)
    assert r["emitted"] == [1] and r["eos"]
    r = K.verify_greedy([10, 11, 12], [11, 12, 13], eos=1, remaining=2)
    assert r["emitted"] == [11, 12] and r["length_limit"]
    with pytest.raises(ValueError):
        K.verify_greedy([1, 2], [2, 3], eos=1, remaining=5)           # anchor is EOS
    with pytest.raises(ValueError):
        K.verify_greedy(list(range(9)), list(range(9)), eos=1000, remaining=5)


# ---------------------------------------------------------------------------------------------- Engram
def test_engram_primes_and_hash_layout():
    p = K.engram_primes()
    assert p[0, 0] == 16000057 and (np.diff(p.reshape(-1).astype(np.int64)) > 0).all()
    h = K.engram_hash([5, 6, 7, 8])
    offs = np.concatenate([[0], np.cumsum(p[0].astype(np.int64))[:-1]])
    assert ((h[0].astype(np.int64) - offs) >= 0).all() and ((h[0].astype(np.int64) - offs) < p[0].astype(np.int64)).all()
    # order-1 columns depend only on the first two tokens
    h2 = K.engram_hash([5, 6, 70, 80])
    assert (h[:, :8] == h2[:, :8]).all() and (h[:, 8:] != h2[:, 8:]).any()


def test_engram_history_is_transactional_and_chunking_invariant():
    toks = list(np.random.default_rng(1).integers(0, 99092, size=12))
    a = K.EngramHistory(pad_id=2)
    whole = a.prepare(toks)
    b = K.EngramHistory(pad_id=2)
    parts = []
    for i in range(0, 12, 5):
        chunk = toks[i:i + 5]
        parts.append(b.prepare(chunk))
        b.commit(chunk, len(chunk))
    assert (np.concatenate(parts) == whole).all() and b.position == 12
    # rejected speculative rows leave no trace
    c = K.EngramHistory(pad_id=2)
    c.commit(toks[:4], 4)
    spec = c.prepare(toks[4:9])
    c.commit(toks[4:9], 2)
    again = c.prepare(toks[6:9])
    assert (again == spec[2:5]).all()
    # image rows (negative ids) hash to zero and reset the lookback
    d = K.EngramHistory(pad_id=2)
    hz = d.prepare([3, -1, 4])
    assert (hz[1] == 0).all() and (hz[2] == K.engram_hash([4, 2, 2, 2])).all()


# ---------------------------------------------------------------------------------------------- prefix banks
def test_prefix_reuse_rule_and_lru():
    banks = K.PrefixBanks(prompt_capacity=2, turn_capacity=2, window=128)
    base = list(range(1000, 1600))
    sid, _ = banks.insert(base, K.PrefixBanks.PROMPT)
    hit = banks.lookup(base + [1, 2, 3])                       # exact ancestor
    assert hit["id"] == sid and hit["exact"] and hit["skipped"] == 600
    hit = banks.lookup(base[:401] + [7, 7, 7])                 # partial: (401//2*2) - 128
    assert hit["id"] == sid and not hit["exact"] and hit["common"] == 401 and hit["skipped"] == 272
    assert banks.lookup(base[:100] + [9]) is None              # too short to pay for the replay window
    assert banks.lookup([5, 6, 7]) is None
    s2, ev = banks.insert([1, 2, 3] * 100, K.PrefixBanks.PROMPT)
    assert ev == -1
    banks.lookup(base)                                          # touch sid -> s2 becomes LRU
    s3, ev = banks.insert([4, 5] * 100, K.PrefixBanks.PROMPT)
    assert ev == s2 and banks.live(0) == 2
    assert banks.lookup([1, 2, 3] * 100) is None
    t1, ev = banks.insert(base + [42], K.PrefixBanks.TURN)      # other bank is independent
    assert ev == -1 and banks.live(1) == 1
    assert banks.lookup(base + [42, 43])["id"] == t1            # longer exact ancestor wins
    assert banks.remove(t1) and not banks.remove(t1)


# ---------------------------------------------------------------------------------------------- KV allocator
def test_kv_leases_pages_and_cow():
    kv = K.KvAllocator(n_pages=8, n_slots=2, page_tokens=64)
    slot, gen = kv.admit()
    new = kv.ensure(slot, gen, 130)
    assert [i for i, _ in new] == [0, 1, 2] and kv.free_pages == 5
    assert kv.ensure(slot, gen, 100) == []
    pages = kv.retain(slot, gen, 2)                              # snapshot keeps two pages
    assert all(kv.page_ref(p) == 2 for p in pages)
    s2, g2 = kv.admit()
    kv.share(s2, g2, pages)
    assert kv.page_count(s2) == 2 and kv.page_ref(pages[0]) == 3
    moved = kv.make_private(s2, g2, 1)                           # copy-on-write before writing page 1
    assert moved is not None and moved[0] == pages[1] and kv.page_ref(pages[1]) == 2
    assert kv.make_private(s2, g2, 1) is None
    with pytest.raises(MemoryError):
        kv.ensure(s2, g2, 64 * 20)
    assert kv.retire(slot, gen) and not kv.retire(slot, gen)     # stale generation rejected
    with pytest.raises(KeyError):
        kv.ensure(slot, gen, 10)
    kv.retire(s2, g2)
    kv.release_pages(pages)
    assert kv.free_pages == 8
    assert kv.admit() is not None and kv.admit() is not None and kv.admit() is None


def test_kv_pool_plan():
    # 64K context, 512-token groups, 16 slots, 20+20 retained snapshots
    want = K.plan_kv_groups(65536, 512, 16, 40, 455680, 1 << 40)
    assert want == 128 * 18 + 16 + 80
    assert K.plan_kv_groups(65536, 512, 16, 40, 455680, 455680 * 100) == 100


def test_philox_vectors_and_reservations():
    """Philox4x32-10 against the published known-answer vector, and forward-only per-request reservations."""
    from ds41rt_b200.runtime import core as K
    # Random123 KAT: counter = key = all ones -> 408f276d 41c83b0e a20bc7c6 6d5451fd
    ones64 = 0xFFFFFFFFFFFFFFFF
    got = [K.philox_uniform(ones64, ones64, ones64, lane) for lane in range(4)]
    want_bits = [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    for g, b in zip(got, want_bits):
        assert g == ((b >> 9) + 0.5) / 8388608.0
    rng = K.DraftRng()
    a = rng.reserve(7, 100)
    b = rng.reserve(7, 50)
    c = rng.reserve(9, 10)
    assert a == (1, 0) and b == (1, 100) and c == (2, 0)
    rng.fork(7, 8)
    assert rng.reserve(8, 5) == (3, 0) and rng.reserve(7, 1) == (1, 150)
    assert rng.release(9) and not rng.release(9)
    rng.close()


def test_kv_allocator_against_a_reference_model_under_random_traffic():
    """Random admissions, growth, snapshots (retain), restores (share), copy-on-write and retirements, mirrored in a
    plain Python model: page reference counts, free-page count and every slot's page list must agree after each step;
    a page is never handed out while something still points at it; stale leases are refused."""
    import random
    rng = random.Random(3)
    N_PAGES, N_SLOTS, P = 24, 4, 16
    kv = K.KvAllocator(N_PAGES, N_SLOTS, page_tokens=P)
    ref = [0] * N_PAGES                                   # model: reference count per page
    slots = {}                                            # slot -> (gen, [pages])
    snaps = []                                            # retained page lists
    stale = []
    steps = {"admit": 0, "grow": 0, "retain": 0, "share": 0, "cow": 0, "retire": 0, "drop": 0, "oom": 0}

    def check():
        assert kv.free_pages == sum(1 for r in ref if r == 0)
        for pg in range(N_PAGES):
            assert kv.page_ref(pg) == ref[pg], pg
        for s, (g, pages) in slots.items():
            assert kv.generation(s) == g and kv.pages(s) == pages
        for s in range(N_SLOTS):
            if s not in slots:
                assert kv.generation(s) == 0 and kv.page_count(s) == 0

    for _ in range(3000):
        op = rng.choice(["admit", "grow", "grow", "retain", "share", "cow", "retire", "drop"])
        if op == "admit":
            got = kv.admit()
            if len(slots) == N_SLOTS:
                assert got is None
            else:
                s, g = got
                assert s not in slots and g != 0
                slots[s] = (g, [])
                steps["admit"] += 1
        elif op == "grow" and slots:
            s = rng.choice(list(slots))
            g, pages = slots[s]
            want = rng.randint(1, 9 * P)
            need = max(0, (want + P - 1) // P - len(pages))
            free = sum(1 for r in ref if r == 0)
            if need > free:
                with pytest.raises(MemoryError):
                    kv.ensure(s, g, want)
                steps["oom"] += 1
            else:
                new = kv.ensure(s, g, want)
                assert len(new) == need
                for idx, pg in new:
                    assert ref[pg] == 0 and idx == len(pages)          # a free page, appended in order
                    ref[pg] = 1
                    pages.append(pg)
                steps["grow"] += 1
        elif op == "retain" and slots:
            s = rng.choice(list(slots))
            g, pages = slots[s]
            n = rng.randint(0, len(pages))
            got = kv.retain(s, g, n)
            assert got == pages[:n]
            for pg in got:
                ref[pg] += 1
            if got:
                snaps.append(got)
            steps["retain"] += 1
        elif op == "share" and snaps:
            empty = [s for s, (g, pages) in slots.items() if not pages]
            if empty:
                s = rng.choice(empty)
                snap = rng.choice(snaps)
                kv.share(s, slots[s][0], snap)
                for pg in snap:
                    ref[pg] += 1
                slots[s] = (slots[s][0], list(snap))
                steps["share"] += 1
        elif op == "cow" and slots:
            s = rng.choice(list(slots))
            g, pages = slots[s]
            if pages:
                i = rng.randrange(len(pages))
                free = sum(1 for r in ref if r == 0)
                if ref[pages[i]] == 1:
                    assert kv.make_private(s, g, i) is None                # already private: nothing to copy
                elif free == 0:
                    with pytest.raises(MemoryError):
                        kv.make_private(s, g, i)
                else:
                    src, dst = kv.make_private(s, g, i)
                    assert src == pages[i] and ref[dst] == 0
                    ref[src] -= 1
                    ref[dst] = 1
                    pages[i] = dst
                    steps["cow"] += 1
        elif op == "retire" and slots:
            s = rng.choice(list(slots))
            g, pages = slots.pop(s)
            assert kv.retire(s, g)
            for pg in pages:
                ref[pg] -= 1
            stale.append((s, g))
            steps["retire"] += 1
        elif op == "drop" and snaps:
            snap = snaps.pop(rng.randrange(len(snaps)))
            kv.release_pages(snap)
            for pg in snap:
                ref[pg] -= 1
            steps["drop"] += 1
        if stale and rng.random() < 0.05:
            s, g = rng.choice(stale)
            if s not in slots or slots[s][0] != g:                         # an old lease of a slot, possibly re-leased
                with pytest.raises(KeyError):
                    kv.ensure(s, g, 1)
                assert not kv.retire(s, g)
        assert all(r >= 0 for r in ref)
        check()
    low = {k: v for k, v in steps.items() if v < 5}
    assert not low, low
