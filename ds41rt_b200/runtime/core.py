"""Python bindings of the host runtime library (libds41_core.so): sampler oracle, speculative verification,
Engram hashing/history, prefix radix banks and the paged KV allocator.  Pure CPU; usable without CUDA."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..ops import lib as _lib

_c = None


def core():
    global _c
    if _c is None:
        c = _lib.core()
        c.ds41_sample_uniform.restype = C.c_float
        c.ds41_sample_uniform.argtypes = [C.c_uint64, C.c_uint64]
        c.ds41_sample_token.restype = C.c_int
        c.ds41_verify_greedy.restype = C.c_int
        for name in ("ds41_engram_history_new", "ds41_engram_history_fork", "ds41_prefix_new", "ds41_kv_new"):
            getattr(c, name).restype = C.c_void_p
        c.ds41_engram_history_position.restype = C.c_uint64
        c.ds41_prefix_insert.restype = C.c_int64
        c.ds41_prefix_lookup.restype = C.c_int64
        c.ds41_kv_plan_groups.restype = C.c_longlong
        _c = c
    return _c


SAMPLE_STATUS = {0: "ok", 1: "empty_candidates", 2: "nonfinite_logit", 3: "invalid_temperature", 4: "mask_width",
                 5: "internal", 6: "invalid_parameter"}


class SamplingError(ValueError):
    pass


def sample_uniform(seed: int, position: int) -> float:
    return float(core().ds41_sample_uniform(seed & (2 ** 64 - 1), position))


def sample_token(logits: np.ndarray, mask: Optional[np.ndarray] = None, temperature: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, min_p: float = 0.0, uniform: float = 0.0) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    tok = C.c_int(-1)
    mp, mw = None, 0
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.uint32)
        mp, mw = mask.ctypes.data_as(C.c_void_p), mask.size
    st = core().ds41_sample_token(logits.ctypes.data_as(C.c_void_p), logits.size, mp, mw, C.c_float(temperature),
                                  int(top_k), C.c_float(top_p), C.c_float(min_p), C.c_float(uniform), C.byref(tok))
    if st != 0:
        raise SamplingError(SAMPLE_STATUS.get(st, str(st)))
    return tok.value


def verify_greedy(inputs: Sequence[int], target_next: Sequence[int], eos: int, remaining: int, vocab: int = 129280):
    n = len(inputs)
    a = (C.c_uint32 * n)(*inputs)
    b = (C.c_uint32 * n)(*target_next)
    out = (C.c_uint32 * n)()
    acc, flags = C.c_int(0), C.c_int(0)
    r = core().ds41_verify_greedy(a, b, n, eos, remaining, vocab, out, C.byref(acc), C.byref(flags))
    if r < 0:
        raise ValueError({-1: "verification requires one to eight corresponding target rows",
                          -2: "completed request cannot verify another anchor",
                          -3: "verification token outside vocabulary"}[r])
    return {"emitted": list(out[:r]), "accepted_inputs": acc.value, "eos": bool(flags.value & 1),
            "length_limit": bool(flags.value & 2)}


# ---------------------------------------------------------------------------------------------- Engram
def engram_primes() -> np.ndarray:
    out = np.zeros((2, 24), dtype=np.uint64)
    core().ds41_engram_primes(out.ctypes.data_as(C.c_void_p))
    return out


def engram_hash(tokens4: Sequence[int]) -> np.ndarray:
    t = (C.c_uint32 * 4)(*tokens4)
    out = np.zeros((2, 24), dtype=np.uint64)
    core().ds41_engram_hash(t, out.ctypes.data_as(C.c_void_p))
    return out


class EngramHistory:
    def __init__(self, pad_id: int = 2, _handle=None):
        self.pad = pad_id
        self.h = C.c_void_p(_handle if _handle is not None else core().ds41_engram_history_new(pad_id))

    def __del__(self):
        try:
            core().ds41_engram_history_free(self.h)
        except Exception:
            pass

    @property
    def position(self) -> int:
        return int(core().ds41_engram_history_position(self.h))

    def fork(self) -> "EngramHistory":
        return EngramHistory(self.pad, core().ds41_engram_history_fork(self.h))

    def prepare(self, tokens: Sequence[int]) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.zeros((len(t), 2, 24), dtype=np.uint64)
        assert core().ds41_engram_prepare(self.h, t.ctypes.data_as(C.c_void_p), len(t),
                                          out.ctypes.data_as(C.c_void_p)) == 0
        return out

    def commit(self, tokens: Sequence[int], accepted: int):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        if core().ds41_engram_commit(self.h, t.ctypes.data_as(C.c_void_p), len(t), accepted) != 0:
            raise ValueError("accepted count outside the prepared batch")


# ---------------------------------------------------------------------------------------------- prefix radix
class PrefixBanks:
    PROMPT, TURN = 0, 1

    def __init__(self, prompt_capacity: int = 20, turn_capacity: int = 20, window: int = 128):
        self.h = C.c_void_p(core().ds41_prefix_new(prompt_capacity, turn_capacity, window))

    def __del__(self):
        try:
            core().ds41_prefix_free(self.h)
        except Exception:
            pass

    def insert(self, tokens: Sequence[int], bank: int = 0) -> Tuple[int, int]:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        ev = C.c_int64(-1)
        sid = core().ds41_prefix_insert(self.h, t.ctypes.data_as(C.c_void_p), len(t), bank, C.byref(ev))
        return int(sid), int(ev.value)

    def remove(self, sid: int) -> bool:
        return core().ds41_prefix_remove(self.h, C.c_int64(sid)) == 0

    def lookup(self, tokens: Sequence[int]):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        common, frontier, skipped = C.c_int(0), C.c_int(0), C.c_int(0)
        sid = core().ds41_prefix_lookup(self.h, t.ctypes.data_as(C.c_void_p), len(t), C.byref(common),
                                        C.byref(frontier), C.byref(skipped))
        if sid < 0:
            return None
        return {"id": int(sid), "common": common.value, "frontier": frontier.value, "skipped": skipped.value,
                "exact": common.value == frontier.value}

    def live(self, bank: int) -> int:
        return int(core().ds41_prefix_live(self.h, bank))

    def oldest(self) -> int:
        """Least recently used live snapshot of either bank, -1 when there is none."""
        core().ds41_prefix_oldest.restype = C.c_int64
        return int(core().ds41_prefix_oldest(self.h))


# ---------------------------------------------------------------------------------------------- KV allocator
class KvAllocator:
    def __init__(self, n_pages: int, n_slots: int, page_tokens: int = 64):
        self.h = C.c_void_p(core().ds41_kv_new(n_pages, n_slots, page_tokens))
        self.page_tokens = page_tokens
        self.n_pages = n_pages

    def __del__(self):
        try:
            core().ds41_kv_free(self.h)
        except Exception:
            pass

    @property
    def free_pages(self) -> int:
        return int(core().ds41_kv_free_pages(self.h))

    def admit(self) -> Optional[Tuple[int, int]]:
        gen = C.c_uint32(0)
        slot = core().ds41_kv_admit(self.h, C.byref(gen))
        return None if slot < 0 else (slot, gen.value)

    def admit_slot(self, slot: int) -> Optional[int]:
        """Take one particular slot -> its generation, or None when it is in use."""
        gen = C.c_uint32(0)
        return gen.value if core().ds41_kv_admit_slot(self.h, slot, C.byref(gen)) == 0 else None

    def generation(self, slot: int) -> int:
        """Generation of an active slot, 0 when the slot is free."""
        core().ds41_kv_slot_generation.restype = C.c_uint32
        return int(core().ds41_kv_slot_generation(self.h, slot))

    def pages(self, slot: int) -> List[int]:
        n = self.page_count(slot)
        if n <= 0:
            return []
        out = (C.c_int32 * n)()
        core().ds41_kv_slot_pages(self.h, slot, out, n)
        return list(out)

    def ensure(self, slot: int, gen: int, n_tokens: int) -> List[Tuple[int, int]]:
        cap = (n_tokens + self.page_tokens - 1) // self.page_tokens + 1
        out = (C.c_int32 * (2 * cap))()
        r = core().ds41_kv_ensure(self.h, slot, gen, n_tokens, out, cap)
        if r == -1:
            raise KeyError("stale lease")
        if r == -2:
            raise MemoryError("KV pool exhausted")
        if r < 0:
            raise ValueError("ensure failed")
        return [(out[2 * i], out[2 * i + 1]) for i in range(r)]

    def share(self, slot: int, gen: int, pages: Sequence[int]):
        a = (C.c_int32 * len(pages))(*pages)
        if core().ds41_kv_share(self.h, slot, gen, a, len(pages)) != 0:
            raise ValueError("share failed")

    def make_private(self, slot: int, gen: int, index: int):
        src, dst = C.c_int32(-1), C.c_int32(-1)
        r = core().ds41_kv_make_private(self.h, slot, gen, index, C.byref(src), C.byref(dst))
        if r < 0:
            raise MemoryError("copy-on-write failed") if r == -2 else KeyError("stale lease or bad index")
        return None if r == 0 else (src.value, dst.value)

    def retain(self, slot: int, gen: int, n_pages: int) -> List[int]:
        out = (C.c_int32 * max(n_pages, 1))()
        r = core().ds41_kv_retain(self.h, slot, gen, n_pages, out)
        if r < 0:
            raise KeyError("stale lease")
        return list(out[:r])

    def release_pages(self, pages: Sequence[int]):
        a = (C.c_int32 * len(pages))(*pages)
        core().ds41_kv_release_pages(self.h, a, len(pages))

    def retire(self, slot: int, gen: int) -> bool:
        return core().ds41_kv_retire(self.h, slot, gen) == 0

    def page_count(self, slot: int) -> int:
        return int(core().ds41_kv_page_count(self.h, slot))

    def page_ref(self, page: int) -> int:
        return int(core().ds41_kv_page_ref(self.h, page))


def plan_kv_groups(ctx: int, group_tokens: int, slots: int, retained: int, bytes_per_group: int, budget: int) -> int:
    return int(core().ds41_kv_plan_groups(C.c_longlong(ctx), group_tokens, slots, retained,
                                          C.c_longlong(bytes_per_group), C.c_longlong(budget)))


# ---------------------------------------------------------------------------------------------- admission / lanes
def _more():
    c = core()
    if not getattr(c, "_ds41_more", False):
        for name in ("ds41_admission_new", "ds41_lanes_new", "ds41_policy_new", "ds41_hostcache_new",
                     "ds41_stubcopy_new"):
            getattr(c, name).restype = C.c_void_p
        c.ds41_policy_acceptance.restype = C.c_double
        c.ds41_stubcopy_copy.restype = C.c_double
        c.ds41_stubcopy_now.restype = C.c_double
        c._ds41_more = True
    return c


class Admission:
    def __init__(self, queue_cap: int, waiter_cap: int):
        self.h = C.c_void_p(_more().ds41_admission_new(queue_cap, waiter_cap))

    def reserve(self) -> int:
        """0 queued, 1 waiting, -1 rejected (HTTP 429)."""
        return int(core().ds41_admission_reserve(self.h))

    def release(self):
        core().ds41_admission_release(self.h)

    def stats(self) -> dict:
        out = (C.c_uint64 * 4)()
        core().ds41_admission_stats(self.h, out)
        return {"queued": out[0], "waiting": out[1], "accepted": out[2], "rejected": out[3]}


class Lanes:
    def __init__(self, n_lanes: int = 2):
        self.n = n_lanes
        self.h = C.c_void_p(_more().ds41_lanes_new(n_lanes))

    def add(self, rid: int, remaining: int, history: int) -> int:
        return int(core().ds41_lanes_add(self.h, C.c_int64(rid), remaining, history))

    def update(self, rid: int, remaining: int, history: int):
        core().ds41_lanes_update(self.h, C.c_int64(rid), remaining, history)

    def retire(self, rid: int) -> int:
        return int(core().ds41_lanes_retire(self.h, C.c_int64(rid)))

    def lane_of(self, rid: int) -> int:
        return int(core().ds41_lanes_lane_of(self.h, C.c_int64(rid)))

    def load(self, lane: int) -> int:
        return int(core().ds41_lanes_load(self.h, lane))

    def plan_round(self, lane: int, draft_len: int, max_rows: int, min_history: int = 0, cap: int = 64):
        ids = (C.c_int64 * cap)()
        rows = (C.c_int * cap)()
        n = core().ds41_lanes_plan_round(self.h, lane, draft_len, max_rows, min_history, ids, rows, cap)
        return [(int(ids[i]), int(rows[i])) for i in range(n)]


class DSparkPolicy:
    def __init__(self, max_width: int = 4, warmup_rounds: int = 12):
        self.h = C.c_void_p(_more().ds41_policy_new(max_width, warmup_rounds))

    def observe(self, width: int, accepted: int, verify_us: float, draft_us: float = 0.0, confidence: float = -1.0):
        core().ds41_policy_observe(self.h, width, accepted, C.c_double(verify_us), C.c_double(draft_us),
                                   C.c_double(confidence))

    def choose(self, confidence: float = -1.0) -> int:
        return int(core().ds41_policy_choose(self.h, C.c_double(confidence)))

    def acceptance(self, depth: int) -> float:
        return float(core().ds41_policy_acceptance(self.h, depth))

    # ---- rounds shared by several requests
    def choose_joint(self, confidences: Sequence[Sequence[float]]) -> List[int]:
        """Verification length of every request of one shared round, from the drafter's confidence in each proposed
        token: maximises expected committed tokens per predicted round time over all requests together."""
        n = len(confidences)
        offs, flat = [0], []
        for c in confidences:
            flat += [float(x) for x in c]
            offs.append(len(flat))
        conf = (C.c_float * max(len(flat), 1))(*flat)
        offsets = (C.c_int * (n + 1))(*offs)
        widths = (C.c_int * max(n, 1))()
        core().ds41_policy_choose_joint(self.h, conf, offsets, n, widths)
        return [int(widths[i]) for i in range(n)]

    def observe_round(self, total_rows: int, n_requests: int, round_us: float):
        core().ds41_policy_observe_round(self.h, total_rows, n_requests, C.c_double(round_us))

    def observe_positions(self, confidence: Sequence[float], width: int, accepted: int):
        """Calibrate the confidence head on every position a verification reached."""
        w = min(width, len(confidence))
        if w > 0:
            core().ds41_policy_observe_positions(self.h, (C.c_float * w)(*[float(x) for x in confidence[:w]]), w,
                                                 min(accepted, w))

    def probe(self, every: int = -1) -> int:
        """Set how often a policy that chose plain decoding answers with a two-draft probe instead (0 = never; -1 leaves
        the cadence as it is); returns the number of probes so far."""
        c = core()
        c.ds41_policy_probe.restype = C.c_uint64
        return int(c.ds41_policy_probe(self.h, every))

    def stats(self) -> dict:
        out = (C.c_double * 8)()
        hist = (C.c_uint64 * 16)()
        core().ds41_policy_stats(self.h, out, hist)
        j = (C.c_double * 6)()
        jc = (C.c_uint64 * 2)()
        core().ds41_policy_joint_stats(self.h, j, jc)
        return {"rounds": int(out[0]), "t_fixed_us": out[1], "t_row_us": out[2], "draft_us_per_row": out[3],
                "platt": [out[4], out[5]], "acceptance_first": out[6], "acceptance_last": out[7],
                "accepted_histogram": list(hist),
                "joint": {"rounds": int(j[5]), "round_fixed_us": j[0], "round_us_per_row": j[1], "fit_weight": j[2],
                          "platt_positions": [j[3], j[4]], "draft_rows_offered": int(jc[0]),
                          "draft_rows_taken": int(jc[1])}}


class HostCache:
    METRICS = ("free_pages", "snapshots", "stored", "shared", "restored", "evictions", "hits", "misses", "deferred",
               "failed")

    def __init__(self, n_pages: int, page_bytes: int, store_budget: int = 1 << 62, restore_budget: int = 1 << 62):
        self.h = C.c_void_p(_more().ds41_hostcache_new(n_pages, C.c_uint64(page_bytes), C.c_uint64(store_budget),
                                                       C.c_uint64(restore_budget)))
        self.page_bytes = page_bytes

    def tick(self):
        core().ds41_hostcache_tick(self.h)

    def store(self, sid: int, keys: Sequence[int], tokens: int = 0):
        n = len(keys)
        k = (C.c_uint64 * n)(*[x & (2 ** 64 - 1) for x in keys])
        pages = (C.c_int32 * n)()
        need = (C.c_uint8 * n)()
        r = core().ds41_hostcache_store(self.h, C.c_int64(sid), k, n, C.c_uint64(tokens), pages, need)
        if r <= 0:
            return r, [], []
        return r, list(pages), [bool(x) for x in need]

    def abort(self, sid: int):
        core().ds41_hostcache_abort(self.h, C.c_int64(sid))

    def restore(self, sid: int, cap: int = 4096):
        pages = (C.c_int32 * cap)()
        r = core().ds41_hostcache_restore(self.h, C.c_int64(sid), pages, cap)
        return r, list(pages[:max(r, 0)])

    def restore_prefix(self, sid: int, n_first: int):
        """The first `n_first` host pages of a snapshot; only they are charged to the restore budget."""
        pages = (C.c_int32 * max(n_first, 1))()
        r = core().ds41_hostcache_restore_prefix(self.h, C.c_int64(sid), n_first, pages, max(n_first, 1))
        return r, list(pages[:max(r, 0)])

    def contains(self, sid: int) -> bool:
        return bool(core().ds41_hostcache_contains(self.h, C.c_int64(sid)))

    def drop(self, sid: int) -> bool:
        return core().ds41_hostcache_drop(self.h, C.c_int64(sid)) == 0

    def metrics(self) -> dict:
        out = (C.c_uint64 * 10)()
        core().ds41_hostcache_metrics(self.h, out)
        return dict(zip(self.METRICS, [int(x) for x in out]))

    def check(self) -> int:
        return int(core().ds41_hostcache_check(self.h))


class StubCopyEngine:
    """Copy engine on a virtual clock (latency + bytes / bandwidth) with one-shot failure injection."""

    def __init__(self, latency_us: float = 10.0, gb_per_s: float = 25.0):
        self.h = C.c_void_p(_more().ds41_stubcopy_new(C.c_double(latency_us), C.c_double(gb_per_s)))

    def fail_at(self, op: int):
        core().ds41_stubcopy_fail_at(self.h, C.c_int64(op))

    def copy(self, nbytes: int) -> float:
        return float(core().ds41_stubcopy_copy(self.h, C.c_uint64(nbytes)))

    @property
    def now_us(self) -> float:
        return float(core().ds41_stubcopy_now(self.h))


def philox_uniform(seed: int, subsequence: int, offset: int, lane: int) -> float:
    """The uniform in (0, 1) that draft sampling uses for token 4 * (offset - base) + lane."""
    c = core()
    c.ds41_philox_uniform.restype = C.c_float
    c.ds41_philox_uniform.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_int]
    return float(c.ds41_philox_uniform(seed & (2 ** 64 - 1), subsequence, offset, lane))


class DraftRng:
    """Per-request Philox subsequences with forward-only counter reservations (csrc/core/rng.cc)."""

    def __init__(self):
        c = core()
        c.ds41_rng_create.restype = C.c_void_p
        c.ds41_rng_destroy.argtypes = [C.c_void_p]
        c.ds41_rng_reserve.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        c.ds41_rng_fork.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64]
        c.ds41_rng_release.argtypes = [C.c_void_p, C.c_uint64]
        self._c, self.h = c, c.ds41_rng_create()

    def reserve(self, request: int, counters: int):
        sub, off = C.c_uint64(0), C.c_uint64(0)
        if self._c.ds41_rng_reserve(self.h, request, counters, C.byref(sub), C.byref(off)) != 0:
            raise ValueError("bad reservation")
        return sub.value, off.value

    def fork(self, parent: int, child: int):
        if self._c.ds41_rng_fork(self.h, parent, child) != 0:
            raise KeyError("unknown parent or existing child")

    def release(self, request: int) -> bool:
        return self._c.ds41_rng_release(self.h, request) == 0

    def close(self):
        if self.h:
            self._c.ds41_rng_destroy(self.h)
            self.h = None
