"""Serving backends: the interface between the HTTP layer and the CUDA-owning worker.

The HTTP threads never touch CUDA.  They put a `GenRequest` on a bounded queue; ONE worker thread owns the
device, runs the scheduler loop (retire -> admit -> prefill -> one batched decode pass -> sample -> emit) and answers
through per-request event queues: Ready(usage) / Tokens / Finish / Error.  A missing Finish is never reported as
success.  (Process layout of the reference: rust/crates/ds41rt-daemon/src/v41_native_serve.rs:73-113,
scheduler.rs:200-451; request/event types: rust/crates/ds41rt-api/src/native_v41.rs:55-65.)

`FakeBackend` scripts token streams for API tests; `NativeBackend` drives a `DS41Engine`.
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np

from ..runtime import core as K
from ..runtime.grammar import TokenConstraint
from .imagekeys import ImageKeySpace
from .protocol import Sampling


@dataclass
class GenRequest:
    prompt_ids: List[int]
    max_tokens: int
    sampling: Sampling
    constraint: Optional[TokenConstraint] = None
    stop_ids: List[int] = field(default_factory=list)
    events: "queue.Queue" = field(default_factory=lambda: queue.Queue())
    cancelled: threading.Event = field(default_factory=threading.Event)
    rid: int = 0
    images: List[Any] = field(default_factory=list)     # (PreparedImage, [prompt positions of its rows]) in order
    image_keys: Any = None    # set at admission: what the prefix banks compare at the image positions (None: not banked)


@dataclass
class Event:
    kind: str                 # ready | tokens | finish | error
    tokens: List[int] = field(default_factory=list)
    reason: str = ""          # finish: stop | length | cancelled
    status: int = 200         # error
    message: str = ""
    usage: Dict[str, int] = field(default_factory=dict)


class Backend:
    healthy = True
    fingerprint = "ds41rt-b200"

    def submit(self, req: GenRequest) -> None:
        raise NotImplementedError

    def stats(self) -> dict:
        return {}

    def close(self) -> None:
        pass


class FakeBackend(Backend):
    """Emits a scripted token list (optionally slowly, or failing midway) - the fake worker of the API tests."""
    fingerprint = "ds41rt-b200-fake"

    def __init__(self, script: Optional[List[int]] = None, tokenizer=None, delay: float = 0.0, fail_after: int = -1,
                 drop_finish: bool = False, chunk: int = 3):
        self.script, self.tk, self.delay, self.fail_after = script, tokenizer, delay, fail_after
        self.drop_finish, self.chunk = drop_finish, chunk
        self.submitted: List[GenRequest] = []
        self.n = 0

    def submit(self, req: GenRequest) -> None:
        self.submitted.append(req)
        self.n += 1
        threading.Thread(target=self._run, args=(req,), daemon=True).start()

    def _run(self, req: GenRequest):
        toks = list(self.script if self.script is not None else [])
        req.events.put(Event("ready", usage={"prompt_tokens": len(req.prompt_ids), "prompt_cache_hit_tokens": 0}))
        sent, reason = 0, "stop"
        for i in range(0, len(toks), self.chunk):
            if req.cancelled.is_set():
                reason = "cancelled"
                break
            if self.fail_after >= 0 and sent >= self.fail_after:
                req.events.put(Event("error", status=500, message="scripted backend failure"))
                return
            part = toks[i:i + self.chunk]
            if sent + len(part) >= req.max_tokens:
                part = part[: req.max_tokens - sent]
                reason = "length"
            if req.constraint is not None:
                for t in part:
                    req.constraint.accept(t)
            req.events.put(Event("tokens", tokens=part))
            sent += len(part)
            if reason == "length":
                break
            if self.delay:
                time.sleep(self.delay)
        if not self.drop_finish:
            req.events.put(Event("finish", reason=reason,
                                 usage={"prompt_tokens": len(req.prompt_ids), "completion_tokens": sent}))

    def stats(self) -> dict:
        return {"requests": self.n}


@dataclass
class _Active:
    req: GenRequest
    slot: int
    gen: int
    pos: int                  # next position to be written
    last: int                 # last emitted token (next input)
    emitted: int = 0
    lane: int = 0
    tokens: List[int] = field(default_factory=list)     # emitted token ids
    spec: bool = False        # the drafter's rings follow this request: it can take part in speculative rounds


@dataclass
class _Prefill:
    """A prompt on its way through the engine, one pass per scheduler iteration (decode rounds of the active requests
    run in between; cancellation is looked at before every pass)."""
    req: GenRequest
    slot: int
    gen: int
    passes: List[tuple]                      # (kind, c0, c1, extra) still to run
    reused: int = 0
    solo: bool = False
    logits: Any = None                       # logits of the prompt's last token once known
    r0: int = 0
    ced: bool = False
    img_rows: Any = None
    img_pos: Any = None
    floor: Optional[int] = None


class NativeBackend(Backend):
    """Worker thread + scheduler loop over a DS41Engine.

    One iteration: retire cancelled requests -> admit queued requests (slot lease, KV pages with snapshot eviction under
    pressure, prefix restore) -> ONE prompt pass of the request being prefilled -> ONE decode round of the active
    requests (captured as a CUDA graph per batch size; greedy rows are selected on the device, sampled or constrained
    rows go through the GPU sampler with the request's allow-mask) -> emit.  With a drafter, a request that is alone on
    the engine is decoded by speculative rounds: greedy unconstrained requests by the all-device round, constrained or
    stochastic ones by a round whose verification rows are selected under per-row grammar masks (a fork of the matcher
    per draft row) or drawn with the request's own (seed, position) numbers and compared with the drafts
    (sample-and-match); the verification-length policy decides per round whether drafting pays.  Up to `spec_lanes`
    active requests share a speculative round: one draft pass proposes a block per request (own slot, rings and Markov
    chain), one target pass verifies all blocks, and each request accepts under its own masks and draws.
    Reference behaviour: rust/crates/ds41rt-daemon/src/v41_native_serve/scheduler.rs:200-451, scheduler/independent.rs,
    constraints.rs:48-68, speculative.rs:121-163."""
    fingerprint = "ds41rt-b200-fp8"

    def __init__(self, engine, eos: int, concurrency: int = 4, queue_depth: int = 16, prefill_chunk: Optional[int] = None,
                 vision=None, drafter=None, engram=None, ced: bool = True, use_graphs: bool = True,
                 prompt_snapshots: int = 20, turn_snapshots: int = 20, host_cache_bytes: int = 0, spec_lanes: int = 4):
        self.e, self.eos = engine, eos
        # prompt passes use the encoder / decoder-replay split when the model has a boundary (config.ced_on)
        self.ced = ced
        self.partial_reuse = True     # snapshots that share only a leading part with a prompt contribute that part
        self.spec = None
        self.policy = None
        # runtime.engram.EngramPipeline or None.  Every pass hands its token ids to the pipeline first (hashes, page
        # advice, gather requests), runs, and commits the rows it kept.  With Engram layers a speculative round reads
        # its drafts back before the target pass (the n-gram hashes of the verification rows need them) and commits
        # only the accepted rows to the slot's history.
        self.engram = engram
        if drafter is not None:
            from ..runtime.speculative import SpecSession
            self.spec = SpecSession(engine, drafter)
            self.policy = K.DSparkPolicy(max_width=self.spec.width - 1)
            # rounds shared by several requests have their own cost model (more rows per pass, one pass for all)
            self.policy_lanes = K.DSparkPolicy(max_width=self.spec.width - 1)
        # how many requests one speculative round can serve (each drafts and verifies its own block in the shared passes)
        self.spec_lanes = max(1, min(spec_lanes, drafter.max_groups)) if drafter is not None else 0
        self.vision = vision                     # models.vision.VisionTower on the engine's device, or None
        self.supports_images = vision is not None
        self.concurrency = min(concurrency, engine.cache.slots, engine.max_rows)
        self.q: "queue.Queue[GenRequest]" = queue.Queue(maxsize=queue_depth)
        self.lanes = K.Lanes(2)
        # Prompt and turn banks: the radix (csrc/core/prefix.cc) owns ids, reuse scores and the per-bank LRU; this map
        # holds what an id stands for: (token tuple, KVSnapshot, logits after the last token or None)
        self.prefix = K.PrefixBanks(prompt_snapshots, turn_snapshots, engine.cfg.window)
        self.snapshots: Dict[int, tuple] = {}
        # pinned-host tier behind the banks: a snapshot that leaves the device (bank eviction, page pressure) is copied
        # there and comes back when a prompt extends it (runtime/hosttier.py)
        self.image_keys = ImageKeySpace()
        self.host_tier = None
        if host_cache_bytes > 0:
            from ..runtime.hosttier import HostSnapshotTier
            self.host_tier = HostSnapshotTier(engine.cache, host_cache_bytes)
        self.prefill_chunk = prefill_chunk or engine.max_rows
        self.active: List[_Active] = []
        self.prefilling: Optional[_Prefill] = None
        self.pending: Optional[GenRequest] = None
        # decode rounds replay one captured graph per batch size; eager when the pass depends on host data per step
        # (Engram rows) or when the engine is a multi-rank mirror (its launches are broadcast call by call)
        self.use_graphs = use_graphs and engram is None and getattr(engine, "group", None) is None \
            and engine.device.type == "cuda"
        self._graphs: Dict[int, Any] = {}
        self._spec_dirty = False
        self.totals = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0, "device_greedy_rows": 0,
                       "cpu_sampled_rows": 0, "gpu_sampled_rows": 0, "rounds": 0, "failed": 0,
                       "prompt_cache_hit_tokens": 0, "snapshots": 0, "spec_rounds": 0, "spec_tokens": 0,
                       "ced_prefills": 0, "partial_prefix_hits": 0, "snapshots_evicted_for_pages": 0,
                       "graph_rounds": 0, "prefill_passes": 0, "spec_masked_rounds": 0, "policy_plain_rounds": 0,
                       "cancelled_in_prefill": 0, "snapshots_demoted": 0, "host_tier_hits": 0, "image_encodes_skipped": 0, "spec_lane_rounds": 0}
        self._rid = 0
        self._stop = threading.Event()
        self._ready = threading.Event()
        self.error: Optional[str] = None
        self.thread = threading.Thread(target=self._worker, name="ds41-cuda-worker", daemon=True)
        self.thread.start()
        self._ready.wait(timeout=120)

    # ------------------------------------------------------------------ HTTP side
    def submit(self, req: GenRequest) -> None:
        if not self.healthy:
            raise RuntimeError("worker is not running")
        self._rid += 1
        req.rid = self._rid
        self.q.put_nowait(req)           # queue.Full -> the HTTP layer answers 429

    def stats(self) -> dict:
        cache = self.e.cache
        out = {"totals": dict(self.totals), "active": len(self.active), "queued": self.q.qsize(),
               "prefilling": self.prefilling is not None,
               "kv": {"pages_free": cache.free_pages, "pages_total": cache.n_pages,
                      "snapshots": len(self.snapshots),
                      "prompt_bank": self.prefix.live(K.PrefixBanks.PROMPT),
                      "turn_bank": self.prefix.live(K.PrefixBanks.TURN)},
               "lanes": [self.lanes.load(0), self.lanes.load(1)],
               "target_sampling": {"device_rounds_rows": self.totals["device_greedy_rows"],
                                   "cpu_fallback_rows": self.totals["cpu_sampled_rows"],
                                   "gpu_sampled_rows": self.totals["gpu_sampled_rows"]}}
        if self.policy is not None:
            out["dspark_policy"] = self.policy.stats()
            out["dspark_policy_shared_rounds"] = self.policy_lanes.stats()
        if self.host_tier is not None:
            out["host_cache"] = self.host_tier.stats()
        if self.supports_images:
            out["image_keys"] = self.image_keys.stats()
        return out

    def close(self) -> None:
        self._stop.set()
        self.thread.join(timeout=30)

    # ------------------------------------------------------------------ worker side
    def _worker(self):
        import torch
        try:
            if self.e.device.type == "cuda":
                torch.cuda.set_device(self.e.device)
            self._ready.set()
            while not self._stop.is_set():
                if self.host_tier is not None:
                    self.host_tier.tick()             # a new scheduler iteration: fresh store / restore budgets
                self._retire()
                self._admit()
                self._prefill_step()
                if not self.active:
                    if self.prefilling is None:
                        time.sleep(0.001)
                    continue
                try:
                    self._decode_round()
                except Exception as ex:           # a failed round fails the active requests; the server keeps running
                    from ..parallel.health import RankFailure
                    if isinstance(ex, RankFailure):
                        for a in self.active:
                            a.req.events.put(Event("error", status=503, message=str(ex)[:300]))
                        raise                     # a rank is gone: this backend cannot launch any more
                    self._device_alive()
                    for a in self.active:
                        a.req.events.put(Event("error", status=500, message=f"decode round failed: {ex}"[:300]))
                        self._release(a.slot, a.req)
                        self.totals["failed"] += 1
                    self.active.clear()
        except Exception as ex:
            self.error = str(ex)
            self.healthy = False
            self._ready.set()

    def _device_alive(self):
        """After a failed pass: a lost CUDA context ends the worker (everything else is the request's problem)."""
        if self.e.device.type == "cuda":
            import torch
            torch.cuda.synchronize(self.e.device)        # raises when the context is gone

    def _engram_pass(self, tokens: List[int], slots: List[int], is_image=None):
        """Start the table reads for one pass and hand the rows to the engine -> pass record to commit afterwards."""
        if self.engram is None:
            return None
        p = self.engram.begin(tokens, slots, is_image)
        self.engram.apply(p, self.e)
        return p

    def _release(self, slot: int, req: GenRequest):
        self.e.cache.release(slot)
        if self.engram is not None:
            self.engram.release(slot)
        self.lanes.retire(req.rid)

    def _fail(self, req: GenRequest, slot: Optional[int], status: int, message: str):
        req.events.put(Event("error", status=status, message=message[:300]))
        if slot is not None:
            self._release(slot, req)
        self.totals["failed"] += 1

    def _finish(self, a: _Active, reason: str):
        self.totals["completion_tokens"] += a.emitted
        if reason in ("stop", "length") and a.emitted > 1 and (not a.req.images or a.req.image_keys is not None):
            # turn bank: the cache holds the prompt and every emitted token but the last one.  Stored before the
            # finish event leaves, so a client that reacts to the event finds the bank as it will stay.
            try:
                self._store_snapshot(a.slot, self._match_ids(a.req, list(a.req.prompt_ids) + a.tokens[:-1]), None,
                                     K.PrefixBanks.TURN)
            except Exception:
                pass
        self._release(a.slot, a.req)
        a.req.events.put(Event("finish", reason=reason, usage={"prompt_tokens": len(a.req.prompt_ids),
                                                               "completion_tokens": a.emitted}))

    def _retire(self):
        keep = []
        for a in self.active:
            if a.req.cancelled.is_set():
                self._finish(a, "cancelled")
            else:
                keep.append(a)
        self.active = keep

    # ------------------------------------------------------------------ admission
    def _slack(self) -> int:
        """Positions a request may touch beyond prompt + max_tokens (speculative rows run ahead of the accepted ones)."""
        return 2 * self.spec.width + 2 if self.spec is not None else 1

    def _ensure_pages(self, slot: int, n_tokens: int) -> bool:
        """Pages for positions [0, n_tokens) of `slot`, dropping least recently used snapshots while the pool is short."""
        while not self.e.cache.ensure(slot, n_tokens):
            if not self._evict_one():
                return False
        return True

    def _evict_one(self) -> bool:
        """Drop the least recently used snapshot (either bank) to free its pages."""
        if not self.snapshots:
            return False
        sid = self.prefix.oldest()
        if sid < 0 or sid not in self.snapshots:
            sid = next(iter(self.snapshots))
        self._drop_snapshot(sid)
        self.totals["snapshots_evicted_for_pages"] += 1
        return True

    def _drop_snapshot(self, sid: int):
        ent = self.snapshots.pop(sid, None)
        self.prefix.remove(sid)
        if ent is not None:
            self._demote(ent)
            self.e.cache.drop_snapshot(ent[1])

    def _demote(self, ent):
        """A snapshot is leaving the device: keep it in host memory when there is a host tier."""
        if self.host_tier is not None:
            toks, snap, logits = ent
            try:
                if self.host_tier.demote(toks, snap, logits):
                    self.totals["snapshots_demoted"] += 1
            except Exception:
                pass                                      # the tier is an optimisation: a failed copy only loses the entry

    def _admit(self):
        while len(self.active) + (1 if self.prefilling is not None else 0) < self.concurrency \
                and self.prefilling is None:
            req = self.pending
            self.pending = None
            if req is None:
                try:
                    req = self.q.get_nowait()
                except queue.Empty:
                    return
            if req.cancelled.is_set():
                continue
            need = len(req.prompt_ids) + req.max_tokens + self._slack()
            if need > self.e.cache.max_ctx:
                req.events.put(Event("error", status=400, message="prompt plus max_tokens exceeds the context window"))
                continue
            lease = self.e.cache.admit()
            if lease is None:
                self.pending = req
                return
            slot, gen = lease
            try:
                parked = self._admit_one(req, slot, gen, need)
            except Exception as ex:
                # the request fails, its slot and pages go back, the worker goes on (unless the device is gone)
                self._fail(req, slot, 503 if isinstance(ex, MemoryError) else 500, f"admission failed: {ex}")
                self._device_alive()
                continue
            if parked:
                return

    def _admit_one(self, req: GenRequest, slot: int, gen: int, need: int) -> bool:
        """Lease pages, restore the best prefix and queue the prompt's passes.  True = parked until a request retires."""
        e = self.e
        if not self._ensure_pages(slot, need):
            e.cache.release(slot)
            if self.active:
                self.pending = req              # park until someone retires
                return True
            req.events.put(Event("error", status=503, message="KV pool cannot hold this request"))
            self.totals["failed"] += 1
            return False
        if req.images:
            req.image_keys = self.image_keys.prepare(req.prompt_ids, req.images)
        reused, snap_logits, replay_from = (0, None, None) if req.images and req.image_keys is None \
            else self._restore_prefix(slot, self._match_ids(req, req.prompt_ids), need)
        first_new = reused
        if replay_from is not None:
            # a truncated snapshot: its compressed rows reach up to the common prefix's even boundary
            first_new = replay_from + e.cfg.window
        req.events.put(Event("ready", usage={"prompt_tokens": len(req.prompt_ids), "prompt_cache_hit_tokens": reused}))
        self.totals["requests"] += 1
        self.totals["prompt_tokens"] += len(req.prompt_ids)
        self.totals["prompt_cache_hit_tokens"] += reused
        # the drafter's rings are fed from this prompt's passes (and from every later pass of the request)
        solo = self.spec is not None and not req.images and req.max_tokens > 1
        self.prefilling = self._plan_prefill(slot, gen, req, first_new, snap_logits, solo, replay_from)
        self.prefilling.reused = reused
        return False

    # ------------------------------------------------------------------ prefix reuse (radix-driven snapshot banks)
    @staticmethod
    def _match_ids(req: GenRequest, tokens: List[int]) -> List[int]:
        """What the banks compare for `tokens` of this request: the tokens themselves, with the placeholder positions of
        every image replaced by that image's key (serving/imagekeys.py).  The model always gets the real tokens."""
        return req.image_keys.encode(tokens) if req.image_keys else tokens

    def _restore_prefix(self, slot: int, prompt: List[int], need: int):
        """Device banks first; a demoted snapshot in the host tier is taken when it reuses more tokens, whether the
        prompt extends it (continued from its end) or only shares a leading part with it (rows up to the cut)."""
        tier = self.host_tier
        hit = tier.lookup(prompt) if tier is not None else None
        part = tier.lookup_partial(prompt) if tier is not None and hit is None and self.partial_reuse else None
        dev_n = 0
        if hit is not None or part is not None:
            dev = self.prefix.lookup(prompt)
            if dev is not None and dev["id"] in self.snapshots:
                dev_n = dev["frontier"] if dev["exact"] else max(0, dev["common"] // 2 * 2 - self.e.cfg.window)
        if part is not None and part[1] > dev_n:
            # only a leading part is shared: its rows come back from the host, the last window before the cut is replayed
            sid, n = part
            self.e.cache.release(slot)
            if self._ensure_pages(slot, n) and tier.restore_prefix_into(slot, sid, n) and self._ensure_pages(slot, need):
                self.totals["host_tier_hits"] += 1
                self.totals["partial_prefix_hits"] += 1
                return n, None, n
            self.e.cache.release(slot)
            if not self._ensure_pages(slot, need):
                raise MemoryError("KV pool cannot hold this request")
        if hit is not None:
            sid, n, has_logits = hit
            usable = n < len(prompt) or (n == len(prompt) and has_logits)
            if usable and n > dev_n:
                self.e.cache.release(slot)
                got = tier.restore_into(slot, sid) if self._ensure_pages(slot, n) else None
                if got is not None and self._ensure_pages(slot, need):
                    self.totals["host_tier_hits"] += 1
                    return n, (got[1] if n == len(prompt) else None), None
                self.e.cache.release(slot)
                if not self._ensure_pages(slot, need):
                    raise MemoryError("KV pool cannot hold this request")
        return self._restore_prefix_device(slot, prompt, need)

    def _restore_prefix_device(self, slot: int, prompt: List[int], need: int):
        """Best stored snapshot for `prompt` -> (tokens reused, logits after them or None, replay start or None).

        The radix names the snapshot and its reuse score.  A snapshot whose tokens are a prefix of the prompt is
        continued from its own end (all of its tokens count).  A snapshot that only shares `common` leading tokens with
        the prompt contributes its compressed rows up to skipped = common / 2 * 2 - window: the windows are rebuilt by
        running the tokens from `skipped` again (third value), so only `skipped` tokens count as reused (reference:
        rust/crates/ds41rt-core/src/prefix.rs:23-30, rust/crates/ds41rt-daemon/src/v41_native_serve/prefix.rs:258-294)."""
        e = self.e
        while True:
            hit = self.prefix.lookup(prompt)
            if hit is None:
                return 0, None, None
            ent = self.snapshots.get(hit["id"])
            if ent is not None:
                break
            self.prefix.remove(hit["id"])                 # the map was cleared behind the radix: forget the id, look again
        toks, snap, logits = ent
        window = e.cfg.window
        n = len(toks)
        exact = hit["exact"] and n <= len(prompt) and not (n == len(prompt) and logits is None)
        score = n if exact else min(hit["common"], len(prompt) - 1) // 2 * 2 - window
        if not exact and (not self.partial_reuse or score <= 0):
            return 0, None, None
        e.cache.release(slot)                             # the slot was given fresh pages by the admission path
        ok = e.cache.restore(slot, snap) if exact else e.cache.restore_prefix(slot, snap, score)
        if not ok:
            # no page for the copied partial page: make room once, else run the whole prompt
            ok = self._evict_one() and (e.cache.restore(slot, snap) if exact
                                        else e.cache.restore_prefix(slot, snap, score))
        if not ok or not self._ensure_pages(slot, need):
            e.cache.release(slot)
            if not self._ensure_pages(slot, need):
                raise MemoryError("KV pool cannot hold this request")
            return 0, None, None
        if exact:
            return n, (logits if n == len(prompt) else None), None
        self.totals["partial_prefix_hits"] += 1
        return score, None, score

    def _store_snapshot(self, slot: int, tokens: List[int], logits, bank: int = 0):
        key = tuple(tokens)
        if not key or any(t == key for t, _, _ in self.snapshots.values()):
            return
        sid, evicted = self.prefix.insert(key, bank)
        if evicted >= 0:
            ent = self.snapshots.pop(evicted, None)
            if ent is not None:
                self._demote(ent)
                self.e.cache.drop_snapshot(ent[1])
        if sid < 0:
            return
        self.snapshots[sid] = (key, self.e.cache.snapshot(slot, len(key)), logits)
        self.totals["snapshots"] += 1

    def _image_rows(self, req: GenRequest, first: int = 0):
        """Run the vision tower over the request's images -> (rows [n, H] bf16, prompt position of every row), or
        (None, None) when no image reaches into the positions from `first` on (all of them restored from a snapshot)."""
        import torch
        rows, positions = [], []
        for image, pos in req.images:
            if pos and max(pos) < first:                      # its rows are in the restored cache already
                self.totals["image_encodes_skipped"] += 1
                continue
            out = self.vision.encode(torch.from_numpy(image.patches), image.grid)
            if out.shape[0] != len(pos):
                raise ValueError("image placeholders do not match the image grid")
            rows.append(out.clone())
            positions += list(pos)
        if not rows:
            return None, None
        return torch.cat(rows, 0).contiguous(), positions

    # ------------------------------------------------------------------ prompt passes, one per scheduler iteration
    def _plan_prefill(self, slot, gen, req, start, logits, solo, replay_from) -> _Prefill:
        """List the passes of a prompt from position `start` on.  With `replay_from` (< start, after a truncated
        snapshot restore) the positions [replay_from, start) run again to rebuild the windows: their compressed rows
        are already in the cache, and every pass of this prompt carries a window floor at `replay_from`."""
        e = self.e
        toks = req.prompt_ids
        pf = _Prefill(req, slot, gen, [], solo=solo, logits=logits, floor=replay_from)
        first = start if replay_from is None else replay_from
        if req.images:
            if self.vision is None:
                raise ValueError("this server has no vision tower")
            pf.img_rows, pf.img_pos = self._image_rows(req, first)     # images below `first` are not encoded again
        if self.engram is not None:
            at = {p for _, pos in req.images for p in pos if p < first}
            self.engram.reset(slot, toks[:first], [i in at for i in range(first)] if at else None)
        end, step = len(toks), self.prefill_chunk
        # passes never straddle `start`: below it the compressed sources are kept, from it on they are produced
        cuts = [(c0, min(hi, c0 + step), hi == end) for lo, hi in ((first, start), (start, end))
                for c0 in range(lo, hi, step)]
        taps_above = (self.spec is None or min(e.cfg.dspark.tap_layers) >= e.cfg.ced_boundary) \
            and e.cfg.ced_replay >= e.cfg.window        # stored snapshots must hold complete decoder windows
        if self.ced and first < end and not req.images and taps_above and e.ced_usable(first, end - first):
            pf.ced, pf.r0 = True, e.ced_replay_start(first, end)
            pf.passes = [("enc", c0, c1, fresh) for c0, c1, fresh in cuts]
            pf.passes += [("replay", c0, min(end, c0 + step), None) for c0 in range(pf.r0, end, step)]
        elif first < end:
            pf.passes = [("full", c0, c1, fresh) for c0, c1, fresh in cuts]
        return pf

    def _prefill_step(self):
        """Run the next pass of the prompt in flight; after its last pass the request joins the decode rounds."""
        pf = self.prefilling
        if pf is None:
            return
        if pf.req.cancelled.is_set():
            self.prefilling = None
            self.totals["cancelled_in_prefill"] += 1
            pf.req.events.put(Event("finish", reason="cancelled",
                                    usage={"prompt_tokens": len(pf.req.prompt_ids), "completion_tokens": 0}))
            self._release(pf.slot, pf.req)
            return
        try:
            if pf.passes:
                self._run_pass(pf, pf.passes.pop(0))
                self.totals["prefill_passes"] += 1
                if pf.passes:
                    return
            self._finish_prefill(pf)
        except Exception as ex:
            self.prefilling = None
            self._fail(pf.req, pf.slot, 503 if isinstance(ex, MemoryError) else 500, f"prompt pass failed: {ex}")
            self._device_alive()

    def _run_pass(self, pf: _Prefill, step):
        import torch
        e, toks, slot = self.e, pf.req.prompt_ids, pf.slot
        kind, c0, c1, extra = step
        self._spec_dirty = True
        m = c1 - c0
        end = len(toks)
        if kind == "enc":
            e.set_rows(toks[c0:c1], list(range(c0, c1)), [slot] * m, row_lo=[pf.floor] * m if pf.floor is not None else None)
            ep = self._engram_pass(toks[c0:c1], [slot] * m)
            e.ced_encoder_slice(c0, c1, pf.r0, extra)
            if ep is not None:
                self.engram.commit(ep)
        elif kind == "replay":
            e.set_rows(toks[c0:c1], list(range(c0, c1)), [slot] * m, row_lo=[pf.r0] * m)
            e.ced_replay_slice(c0, c1, pf.r0, c1 >= end)
            if pf.solo:
                self.spec.d.feed(m)
        else:
            part = toks[c0:c1]
            image_at = set(pf.img_pos) if pf.img_pos is not None else set()
            e.set_rows(part, list(range(c0, c1)), [slot] * m, row_lo=[pf.floor] * m if pf.floor is not None else None)
            ep = self._engram_pass(part, [slot] * m, [c0 + i in image_at for i in range(m)])
            if pf.img_rows is not None:
                ids = [p - c0 if c0 <= p < c1 else -1 for p in pf.img_pos]
                if any(i >= 0 for i in ids):
                    e.image_patch = (pf.img_rows, torch.tensor(ids, dtype=torch.int32, device=pf.img_rows.device))
            try:
                e.forward_rows(m, head=c1 >= end, sources=extra)
            finally:
                e.image_patch = None
            if ep is not None:
                self.engram.commit(ep)
            if pf.solo:
                self.spec.d.feed(m)           # the drafter's rings follow the target's taps

    def _finish_prefill(self, pf: _Prefill):
        e, req, slot = self.e, pf.req, pf.slot
        self.prefilling = None
        if pf.logits is None:
            pf.logits = e.logits_rows(e.last_head_row + 1)[e.last_head_row].clone()
            if pf.ced:
                self.totals["ced_prefills"] += 1
            if not req.images or req.image_keys is not None:  # image prompts are banked under their image keys
                self._store_snapshot(slot, self._match_ids(req, req.prompt_ids), pf.logits, K.PrefixBanks.PROMPT)
        first = self._select([req], [0], logits=pf.logits.view(1, -1))[0]
        a = _Active(req, slot, pf.gen, pos=len(req.prompt_ids), last=first, spec=pf.solo)
        if pf.solo and not self.active and req.sampling.greedy and req.constraint is None:
            self.spec.prime(slot, first, len(req.prompt_ids))
        a.lane = self.lanes.add(req.rid, req.max_tokens, len(req.prompt_ids))
        if self._emit(a, first):
            self.active.append(a)

    # ------------------------------------------------------------------ selection
    def _select(self, reqs: List[GenRequest], rows: List[int], logits=None, positions=None, masks=None) -> List[int]:
        """Pick the next token of each request from the logits row it owns in the last pass (or in `logits`).
        `positions`: sampling position per row (default: the request's emitted count); `masks`: allow-mask per row
        (default: the request's constraint as it stands)."""
        import torch
        e = self.e
        out = []
        simple = logits is None and masks is None and all(r.sampling.greedy and r.constraint is None for r in reqs)
        if simple:
            chosen = e.chosen.tolist()
            self.totals["device_greedy_rows"] += len(reqs)
            return [chosen[i] for i in rows]
        # sampled or grammar-constrained rows: the GPU sampler reads the logits where they are; only the packed
        # allow-masks (vocab/8 bytes per constrained row) go up and one token id per row comes back
        from ..ops.sampling import RowParams, pack_params, sample_rows
        if logits is None:
            logits = e.logits_rows(max(rows) + 1)
        if logits.dtype != torch.float32:
            logits = logits.float()
        picked = logits[torch.tensor(rows, device=logits.device)] if rows != list(range(len(rows))) else logits[:len(rows)]
        params, arena_rows = [], []
        for i, r in enumerate(reqs):
            s = r.sampling
            mask_row = -1
            m = masks[i] if masks is not None else (r.constraint.mask() if r.constraint is not None else None)
            if m is not None:
                mask_row = len(arena_rows)
                arena_rows.append(np.ascontiguousarray(m, dtype=np.uint32))
            position = positions[i] if positions is not None else getattr(r, "_emitted", 0)
            params.append(RowParams(temperature=0.0 if s.greedy else s.temperature, top_k=s.top_k, top_p=s.top_p,
                                    min_p=s.min_p, seed=s.seed, position=position, mask_row=mask_row))
        arena = None
        if arena_rows:
            arena = torch.from_numpy(np.stack(arena_rows).view(np.int32)).to(logits.device)
        toks, status = sample_rows(picked.contiguous(), pack_params(params, logits.device), arena)
        toks, status = toks.tolist(), status.tolist()
        for r, tok, st in zip(reqs, toks, status):
            if st != 0:
                # the oracle names the failure (no candidate under the mask, non-finite logits, bad parameters)
                raise K.SamplingError(K.SAMPLE_STATUS.get(st, str(st)))
            out.append(tok)
            self.totals["gpu_sampled_rows"] += 1
        e.check_status("serving pass")
        return out

    def _emit(self, a: _Active, tok: int) -> bool:
        """Deliver one token; returns False when the request finished."""
        r = a.req
        if r.constraint is not None and not r.constraint.accept(tok):
            r.events.put(Event("error", status=500, message="selected token violates the request's grammar"))
            self._release(a.slot, r)
            return False
        a.emitted += 1
        a.tokens.append(tok)
        r._emitted = a.emitted
        a.last = tok
        if tok == self.eos or tok in r.stop_ids:
            self._finish(a, "stop")
            return False
        r.events.put(Event("tokens", tokens=[tok]))
        if a.emitted >= r.max_tokens:
            self._finish(a, "length")
            return False
        if r.constraint is not None and r.constraint.matcher is not None and not r.constraint.in_thinking \
                and r.constraint.matcher.terminated:
            self._finish(a, "stop")
            return False
        return True

    # ------------------------------------------------------------------ speculative rounds (one request on the engine)
    def _spec_round(self, a: _Active, gate: int = 0):
        """One speculative round for the only active request: up to `width` tokens come back."""
        import torch
        r = a.req
        plain = r.sampling.greedy and r.constraint is None and self.engram is None
        timed = self.e.device.type == "cuda"
        if timed:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        if plain:
            if self._spec_dirty:                   # another request's prompt pass used the engine's input rows
                self.spec.prime(a.slot, a.last, a.pos)
                self._spec_dirty = False
            toks = self.spec.round_host()
            drafts_checked = self.spec.width - 1
        else:
            toks, drafts_checked = self._spec_round_selected(a, gate)
            self.totals["spec_masked_rounds"] += 1
        us = -1.0                                  # no device clock (a CPU engine): only the acceptance is observed
        if timed:
            ev1.record()
            ev1.synchronize()
            us = ev0.elapsed_time(ev1) * 1e3
        conf = self.spec.last_confidence
        self.policy.observe(drafts_checked, max(0, len(toks) - 1), us, confidence=conf[0] if conf else -1.0)
        self.totals["rounds"] += 1
        self.totals["spec_rounds"] += 1
        self.totals["spec_tokens"] += len(toks)
        keep = True
        for t in toks:
            a.pos += 1
            if not self._emit(a, t):
                keep = False
                break
        if keep:
            self.lanes.update(a.req.rid, a.req.max_tokens - a.emitted, a.pos)
        self.active = [a] if keep else []

    def _spec_round_selected(self, a: _Active, gate: int = 0):
        """Speculative round whose verification rows are selected on the host's terms: drafts come back first, the
        proposal is cut at the first token the grammar rejects, every verification row gets the mask of a matcher fork
        advanced over the drafts before it, and the rows are drawn by the GPU sampler with the request's own
        (seed, position) numbers - a draft counts while it equals the target's own draw (sample-and-match)."""
        r, sp, e = a.req, self.spec, self.e
        w = sp.width
        drafts = sp.draft_host(a.slot, a.last, a.pos)                    # w - 1 proposed tokens
        if sp.last_confidence:
            # verification length from the policy, given how sure the drafter is of its first token
            # (`gate` > 0: the policy opened this round as a probe, whose width is kept)
            drafts = drafts[: max(self.policy.choose(sp.last_confidence[0]), gate, 0)]
        if r.constraint is not None:
            drafts = r.constraint.truncate_proposal(drafts)
        remaining = r.max_tokens - a.emitted
        drafts = drafts[: max(0, min(len(drafts), remaining - 1))]
        inputs = [a.last] + drafts
        n = len(inputs)
        masks = r.constraint.row_masks(inputs) if r.constraint is not None else None
        ep = self._engram_pass(inputs, [a.slot] * n)                     # table rows of the n verification rows
        sp.verify_host(a.slot, inputs, a.pos)                            # target pass over the n rows, rings fed
        picked = self._select([r] * n, list(range(n)), positions=[a.emitted + i for i in range(n)], masks=masks)
        accepted = 0
        while accepted < n - 1 and picked[accepted] == drafts[accepted] and picked[accepted] != self.eos \
                and picked[accepted] not in r.stop_ids:
            accepted += 1
        if ep is not None:
            self.engram.commit(ep, {a.slot: accepted + 1})               # the anchor and the accepted drafts
        return picked[: accepted + 1], len(drafts)

    def _spec_round_lanes(self, acts: List[_Active], gate: int = 0):
        """One speculative round shared by several requests: one draft pass proposes a block per request, each proposal
        is cut by the policy (given the drafter's confidence in it), by the request's grammar and by its token budget,
        one target pass verifies all blocks, and every request keeps the drafts that equal the target's own selection
        under its own sampling parameters and row masks, plus the bonus token."""
        import torch
        sp = self.spec
        timed = self.e.device.type == "cuda"
        if timed:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        proposals, confs = sp.draft_host_groups([a.slot for a in acts], [a.last for a in acts], [a.pos for a in acts])
        inputs, masks, reqs, positions, slots_rows, toks_rows = [], [], [], [], [], []
        # with a confidence head the lengths of all requests are chosen together (one pass pays for all rows)
        widths = self.policy_lanes.choose_joint([c[: len(d)] for d, c in zip(proposals, confs)]) \
            if confs and all(confs) else None
        for i, (a, drafts, conf) in enumerate(zip(acts, proposals, confs)):
            r = a.req
            if widths is not None:
                drafts = drafts[: max(widths[i], gate, 0)]
            if r.constraint is not None:
                drafts = r.constraint.truncate_proposal(drafts)
            drafts = drafts[: max(0, min(len(drafts), r.max_tokens - a.emitted - 1))]
            inp = [a.last] + drafts
            inputs.append(inp)
            row_masks = r.constraint.row_masks(inp) if r.constraint is not None else [None] * len(inp)
            masks += row_masks
            reqs += [r] * len(inp)
            positions += [a.emitted + i for i in range(len(inp))]
            slots_rows += [a.slot] * len(inp)
            toks_rows += inp
        ep = self._engram_pass(toks_rows, slots_rows)
        first = sp.verify_host_groups([a.slot for a in acts], inputs, [a.pos for a in acts])
        n_rows = len(toks_rows)
        picked = self._select(reqs, list(range(n_rows)), positions=positions,
                              masks=masks if any(m is not None for m in masks) else None)
        accepted = []
        for a, inp, f in zip(acts, inputs, first):
            r, k = a.req, 0
            while k < len(inp) - 1 and picked[f + k] == inp[k + 1] and picked[f + k] != self.eos \
                    and picked[f + k] not in r.stop_ids:
                k += 1
            accepted.append(k)
        if ep is not None:
            self.engram.commit(ep, {a.slot: k + 1 for a, k in zip(acts, accepted)})
        share = -1.0
        if timed:
            ev1.record()
            ev1.synchronize()
            share = ev0.elapsed_time(ev1) * 1e3 / len(acts)
        for inp, k, conf in zip(inputs, accepted, confs):
            self.policy_lanes.observe(len(inp) - 1, k, share, confidence=conf[0] if conf else -1.0)
            if conf:
                self.policy_lanes.observe_positions(conf, len(inp) - 1, k)
        if timed:
            self.policy_lanes.observe_round(n_rows, len(acts), share * len(acts))
        self.totals["rounds"] += 1
        self.totals["spec_rounds"] += 1
        self.totals["spec_lane_rounds"] += 1
        self._spec_dirty = True                      # the all-device round of a lone request starts from fresh inputs
        keep = []
        for a, f, k in zip(acts, first, accepted):
            alive = True
            self.totals["spec_tokens"] += k + 1
            for t in picked[f: f + k + 1]:
                a.pos += 1
                if not self._emit(a, t):
                    alive = False
                    break
            if alive:
                self.lanes.update(a.req.rid, a.req.max_tokens - a.emitted, a.pos)
                keep.append(a)
        self.active = keep

    @staticmethod
    def _gate(policy):
        """(verification width the policy wants before drafting, whether that answer is one of its periodic probes).  A
        probe's width is handed to the round, whose second look at the policy - with the drafter's confidence - would
        otherwise cut the proposal to nothing and leave the probe without an observation."""
        before = policy.probe()
        width = policy.choose()
        return width, policy.probe() > before

    # ------------------------------------------------------------------ decode rounds
    def _graph_for(self, rows: int):
        """Captured launch sequence of one `rows`-row decode pass (made on first use of a batch size)."""
        import torch
        g = self._graphs.get(rows)
        if g is None:
            e = self.e
            keep = (e.in_tokens.clone(), e.row_pos.clone(), e.row_slot.clone())
            e.forward_rows(rows)                      # eager pass first: kernel attributes, every code path warm
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                e.forward_rows(rows)
            e.in_tokens.copy_(keep[0])
            e.row_pos.copy_(keep[1])
            e.row_slot.copy_(keep[2])
            self._graphs[rows] = g
        return g

    def _decode_round(self):
        e = self.e
        acts = self.active
        if len(acts) == 1 and acts[0].spec:
            a = acts[0]
            gate, probe = self._gate(self.policy) if a.req.max_tokens - a.emitted > 1 else (0, False)
            if gate > 0:
                return self._spec_round(a, gate if probe else 0)
            self.totals["policy_plain_rounds"] += 1
        elif 1 < len(acts) <= self.spec_lanes and all(a.spec for a in acts) \
                and (len(acts) + 1) * self.spec.width <= e.max_rows:
            gate, probe = self._gate(self.policy_lanes)
            if gate > 0:
                return self._spec_round_lanes(acts, gate if probe else 0)
            self.totals["policy_plain_rounds"] += 1
        e.set_rows([a.last for a in acts], [a.pos for a in acts], [a.slot for a in acts])
        if self.use_graphs:
            self._graph_for(len(acts)).replay()
            self.totals["graph_rounds"] += 1
        else:
            ep = self._engram_pass([a.last for a in acts], [a.slot for a in acts])
            e.forward_rows(len(acts))
            if ep is not None:
                self.engram.commit(ep)
        if self.spec is not None and any(a.spec for a in acts):
            self.spec.d.feed(len(acts))             # the drafter's rings follow a plain step too
            self._spec_dirty = self._spec_dirty or len(acts) > 1
        toks = self._select([a.req for a in acts], list(range(len(acts))))
        self.totals["rounds"] += 1
        keep = []
        for a, t in zip(acts, toks):
            a.pos += 1
            self.lanes.update(a.req.rid, a.req.max_tokens - a.emitted, a.pos)
            if self._emit(a, t):
                keep.append(a)
        self.active = keep
        if len(keep) == 1 and keep[0].spec and keep[0].req.sampling.greedy and keep[0].req.constraint is None:
            self.spec.prime(keep[0].slot, keep[0].last, keep[0].pos)      # the all-device round starts from here
