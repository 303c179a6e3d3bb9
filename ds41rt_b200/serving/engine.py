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
    spec: bool = False        # decoded by speculative rounds (drafter + verify) while it is the only active request


class NativeBackend(Backend):
    """Worker thread + scheduler loop over a DS41Engine (target-only batched decode; greedy rows are selected on
    the device, sampled or constrained rows go through the GPU sampler with the request's allow-mask).  With a
    drafter, a greedy unconstrained request that is alone on the engine is decoded by speculative rounds (dSpark drafts,
    one verification pass, device-side accept rule); it drops to plain decoding when a second request joins."""
    fingerprint = "ds41rt-b200-fp8"

    def __init__(self, engine, eos: int, concurrency: int = 4, queue_depth: int = 16, prefill_chunk: Optional[int] = None,
                 vision=None, drafter=None, engram=None, ced: bool = True):
        self.e, self.eos = engine, eos
        # prompt passes use the encoder / decoder-replay split when the model has a boundary (config.ced_on)
        self.ced = ced
        self.partial_reuse = True     # snapshots that share only a leading part with a prompt contribute that part
        self.spec = None
        # runtime.engram.EngramPipeline or None.  Every pass hands its token ids to the pipeline first (hashes, page
        # advice, gather requests), runs, and commits the rows it kept.  Speculative rounds keep their draft tokens on
        # the device, so a backend with Engram layers decodes without the drafter.
        self.engram = engram
        if engram is not None:
            drafter = None
        if drafter is not None:
            from ..runtime.speculative import SpecSession
            self.spec = SpecSession(engine, drafter)
        self.vision = vision                     # models.vision.VisionTower on the engine's device, or None
        self.supports_images = vision is not None
        self.concurrency = min(concurrency, engine.cache.slots, engine.max_rows)
        self.q: "queue.Queue[GenRequest]" = queue.Queue(maxsize=queue_depth)
        self.kv = K.KvAllocator(engine.cache.n_pages, engine.cache.slots, engine.cache.page_tokens)
        self.lanes = K.Lanes(2)
        self.prefix = K.PrefixBanks(20, 20, engine.cfg.window)
        # KV snapshots at prompt ends and turn ends, newest last: (token tuple, KVSnapshot, logits after the last token)
        self.snapshots: List[tuple] = []
        self.snapshot_capacity = 40
        self.prefill_chunk = prefill_chunk or engine.max_rows
        self.active: List[_Active] = []
        self.pending: Optional[GenRequest] = None
        self.totals = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0, "device_greedy_rows": 0,
                       "cpu_sampled_rows": 0, "gpu_sampled_rows": 0, "rounds": 0, "failed": 0,
                       "prompt_cache_hit_tokens": 0, "snapshots": 0, "spec_rounds": 0, "spec_tokens": 0,
                       "ced_prefills": 0, "partial_prefix_hits": 0}
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
        pages_free = self.kv.free_pages
        return {"totals": dict(self.totals), "active": len(self.active), "queued": self.q.qsize(),
                "kv": {"pages_free": pages_free, "pages_total": self.kv.n_pages},
                "lanes": [self.lanes.load(0), self.lanes.load(1)],
                "target_sampling": {"device_rounds_rows": self.totals["device_greedy_rows"],
                                    "cpu_fallback_rows": self.totals["cpu_sampled_rows"],
                                    "gpu_sampled_rows": self.totals["gpu_sampled_rows"]}}

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
                self._retire()
                self._admit()
                if not self.active:
                    time.sleep(0.001)
                    continue
                try:
                    self._decode_round()
                except Exception as ex:           # a failed round fails the active requests; the server keeps running
                    for a in self.active:
                        a.req.events.put(Event("error", status=500, message=f"decode round failed: {ex}"[:300]))
                        self._release(a)
                        self.totals["failed"] += 1
                    self.active.clear()
        except Exception as ex:
            self.error = str(ex)
            self.healthy = False
            self._ready.set()

    def _engram_pass(self, tokens: List[int], slots: List[int], is_image=None):
        """Start the table reads for one pass and hand the rows to the engine -> pass record to commit afterwards."""
        if self.engram is None:
            return None
        p = self.engram.begin(tokens, slots, is_image)
        self.engram.apply(p, self.e)
        return p

    def _release(self, a: _Active):
        self.kv.retire(a.slot, a.gen)
        self.e.cache.release(a.slot)
        if self.engram is not None:
            self.engram.release(a.slot)
        self.lanes.retire(a.req.rid)

    def _finish(self, a: _Active, reason: str):
        a.req.events.put(Event("finish", reason=reason, usage={"prompt_tokens": len(a.req.prompt_ids),
                                                               "completion_tokens": a.emitted}))
        self.totals["completion_tokens"] += a.emitted
        if reason in ("stop", "length") and a.emitted > 1 and not a.req.images:
            # turn bank: the cache holds the prompt and every emitted token but the last one
            try:
                self._store_snapshot(a.slot, list(a.req.prompt_ids) + a.tokens[:-1], None)
            except Exception:
                pass
        self._release(a)

    def _retire(self):
        keep = []
        for a in self.active:
            if a.req.cancelled.is_set():
                self._finish(a, "cancelled")
            else:
                keep.append(a)
        self.active = keep

    def _admit(self):
        while len(self.active) < self.concurrency:
            req = self.pending
            self.pending = None
            if req is None:
                try:
                    req = self.q.get_nowait()
                except queue.Empty:
                    return
            if req.cancelled.is_set():
                continue
            need = len(req.prompt_ids) + req.max_tokens + 1
            if need > self.e.cache.max_ctx:
                req.events.put(Event("error", status=400, message="prompt plus max_tokens exceeds the context window"))
                continue
            lease = self.kv.admit()
            if lease is None:
                self.pending = req
                return
            slot, gen = lease
            try:
                self.kv.ensure(slot, gen, need)
            except MemoryError:
                self.kv.retire(slot, gen)
                if self.active:
                    self.pending = req          # park until someone retires
                    return
                req.events.put(Event("error", status=503, message="KV pool cannot hold this request"))
                continue
            if not self.e.cache.ensure(slot, need):
                self.kv.retire(slot, gen)
                req.events.put(Event("error", status=503, message="KV pool cannot hold this request"))
                continue
            self.prefix.lookup(req.prompt_ids)
            reused, snap_logits, replay_from = (0, None, None) if req.images \
                else self._restore_prefix(slot, req.prompt_ids)
            first_new = reused
            if replay_from is not None:
                # a truncated snapshot: its compressed rows reach up to the common prefix's even boundary
                first_new = replay_from + self.e.cfg.window
            req.events.put(Event("ready", usage={"prompt_tokens": len(req.prompt_ids),
                                                 "prompt_cache_hit_tokens": reused}))
            self.totals["requests"] += 1
            self.totals["prompt_tokens"] += len(req.prompt_ids)
            self.totals["prompt_cache_hit_tokens"] += reused
            solo = (self.spec is not None and not self.active and req.sampling.greedy and req.constraint is None
                    and not req.images and req.max_tokens > 1)
            first = self._prefill(slot, req, start=first_new, logits=snap_logits, feed_drafter=solo,
                                  replay_from=replay_from)
            a = _Active(req, slot, gen, pos=len(req.prompt_ids), last=first, spec=solo)
            if solo:
                self.spec.prime(slot, first, len(req.prompt_ids))
            a.lane = self.lanes.add(req.rid, req.max_tokens, len(req.prompt_ids))
            self.prefix.insert(req.prompt_ids, K.PrefixBanks.PROMPT)
            if self._emit(a, first):
                self.active.append(a)

    # ------------------------------------------------------------------ prefix reuse (exact snapshot boundaries)
    def _restore_prefix(self, slot: int, prompt: List[int]):
        """Best stored snapshot for `prompt` -> (tokens reused, logits after them or None, replay start or None).

        A snapshot whose tokens are a prefix of the prompt is continued from its own end (all of its tokens count).  A
        snapshot that only shares `common` leading tokens with the prompt contributes its compressed rows up to
        skipped = common / 2 * 2 - window: the windows are rebuilt by running the tokens from `skipped` again (third
        value), so only `skipped` tokens count as reused.  The higher count wins (reference:
        rust/crates/ds41rt-core/src/prefix.rs:23-30, rust/crates/ds41rt-daemon/src/v41_native_serve/prefix.rs:258-294)."""
        window = self.e.cfg.window
        best, best_score, best_exact = None, 0, False
        for i, (toks, snap, logits) in enumerate(self.snapshots):
            n = len(toks)
            common = 0
            for a, b in zip(toks, prompt):
                if a != b:
                    break
                common += 1
            if common == n and n <= len(prompt):
                if n == len(prompt) and logits is None:
                    continue                               # nothing to continue from without the last logits
                score, exact = n, True
            else:
                score, exact = common // 2 * 2 - window, False
                if not self.partial_reuse or score <= 0 or common >= len(prompt):
                    continue
            if score > best_score:
                best, best_score, best_exact = i, score, exact
        if best is None:
            return 0, None, None
        toks, snap, logits = self.snapshots[best]
        self.e.cache.release(slot)                     # the slot was given fresh pages by the admission path
        if best_exact:
            if not self.e.cache.restore(slot, snap):
                self.e.cache.ensure(slot, len(prompt) + 1)
                return 0, None, None
            self.snapshots.append(self.snapshots.pop(best))   # most recently used last
            return len(toks), (logits if len(toks) == len(prompt) else None), None
        if not self.e.cache.restore_prefix(slot, snap, best_score):
            self.e.cache.ensure(slot, len(prompt) + 1)
            return 0, None, None
        self.snapshots.append(self.snapshots.pop(best))
        self.totals["partial_prefix_hits"] += 1
        return best_score, None, best_score

    def _store_snapshot(self, slot: int, tokens: List[int], logits):
        key = tuple(tokens)
        if not key or any(t == key for t, _, _ in self.snapshots):
            return
        self.snapshots.append((key, self.e.cache.snapshot(slot, len(key)), logits))
        self.totals["snapshots"] += 1
        while len(self.snapshots) > self.snapshot_capacity:
            _, old, _ = self.snapshots.pop(0)
            self.e.cache.drop_snapshot(old)

    def _image_rows(self, req: GenRequest):
        """Run the vision tower over the request's images -> (rows [n, H] bf16, prompt position of every row)."""
        import torch
        rows, positions = [], []
        for image, pos in req.images:
            out = self.vision.encode(torch.from_numpy(image.patches), image.grid)
            if out.shape[0] != len(pos):
                raise ValueError("image placeholders do not match the image grid")
            rows.append(out.clone())
            positions += list(pos)
        return torch.cat(rows, 0).contiguous(), positions

    def _prefill(self, slot: int, req: GenRequest, start: int = 0, logits=None, feed_drafter: bool = False,
                 replay_from: Optional[int] = None) -> int:
        """Run the prompt from position `start` on.  With `replay_from` (< start, after a truncated snapshot restore)
        the positions [replay_from, start) are run again to rebuild the windows: their compressed rows are already in
        the cache, and every pass of this prompt carries a window floor at `replay_from`."""
        import torch
        e = self.e
        toks = req.prompt_ids
        img_rows = img_pos = None
        if req.images:
            if self.vision is None:
                raise ValueError("this server has no vision tower")
            img_rows, img_pos = self._image_rows(req)
        slack = 2 * self.spec.width + 2 if self.spec is not None else 1
        if not e.cache.ensure(slot, len(toks) + req.max_tokens + slack):
            raise MemoryError("KV pool cannot hold this request")
        first = start if replay_from is None else replay_from
        if self.engram is not None:
            self.engram.reset(slot, toks[:first])
        image_at = set(img_pos) if img_pos is not None else set()
        end, step = len(toks), self.prefill_chunk
        # passes never straddle `start`: below it the compressed sources are kept, from it on they are produced
        cuts = [(c0, min(hi, c0 + step), hi == end) for lo, hi in ((first, start), (start, end))
                for c0 in range(lo, hi, step)]
        floor = (lambda m: [replay_from] * m) if replay_from is not None else (lambda m: None)
        taps_above = (self.spec is None or min(e.cfg.dspark.tap_layers) >= e.cfg.ced_boundary) \
            and e.cfg.ced_replay >= e.cfg.window        # stored snapshots must hold complete decoder windows
        if self.ced and first < end and not req.images and taps_above and e.ced_usable(first, end - first):
            # encoder slices over the new tokens, then the decoder layers over the tail only
            r0 = e.ced_replay_start(first, end)
            for c0, c1, fresh in cuts:
                e.set_rows(toks[c0:c1], list(range(c0, c1)), [slot] * (c1 - c0), row_lo=floor(c1 - c0))
                ep = self._engram_pass(toks[c0:c1], [slot] * (c1 - c0))
                e.ced_encoder_slice(c0, c1, r0, fresh)
                if ep is not None:
                    self.engram.commit(ep)
            for c0 in range(r0, end, step):
                c1 = min(end, c0 + step)
                e.set_rows(toks[c0:c1], list(range(c0, c1)), [slot] * (c1 - c0), row_lo=[r0] * (c1 - c0))
                e.ced_replay_slice(c0, c1, r0, c1 >= end)
                if feed_drafter:
                    self.spec.d.feed(c1 - c0)
            self.totals["ced_prefills"] += 1
            logits = e.logits_rows(e.last_head_row + 1)[e.last_head_row].clone()
            self._store_snapshot(slot, toks, logits)
        elif first < end:
            for c0, c1, fresh in cuts:
                part = toks[c0:c1]
                e.set_rows(part, list(range(c0, c1)), [slot] * len(part), row_lo=floor(len(part)))
                ep = self._engram_pass(part, [slot] * len(part), [c0 + i in image_at for i in range(len(part))])
                last = c1 >= end
                if img_rows is not None:
                    ids = [p - c0 if c0 <= p < c1 else -1 for p in img_pos]
                    if any(i >= 0 for i in ids):
                        e.image_patch = (img_rows, torch.tensor(ids, dtype=torch.int32, device=img_rows.device))
                e.forward_rows(len(part), head=last, sources=fresh)
                e.image_patch = None
                if ep is not None:
                    self.engram.commit(ep)
                if feed_drafter:
                    self.spec.d.feed(len(part))       # the drafter's rings follow the target's taps
            logits = e.logits_rows(e.last_head_row + 1)[e.last_head_row].clone()
            if not req.images:                                # placeholders look alike: image prompts are not banked
                self._store_snapshot(slot, toks, logits)      # prompt bank
        return self._select([req], [0], logits=logits.view(1, -1))[0]

    def _select(self, reqs: List[GenRequest], rows: List[int], logits=None) -> List[int]:
        """Pick the next token of each request from the logits row it owns in the last pass (or in `logits`)."""
        import torch
        e = self.e
        out = []
        simple = logits is None and all(r.sampling.greedy and r.constraint is None for r in reqs)
        if simple:
            chosen = e.chosen.tolist()
            self.totals["device_greedy_rows"] += len(reqs)
            return [chosen[i] for i in rows]
        # sampled or grammar-constrained rows: the GPU sampler reads the logits where they are; only the packed
        # allow-masks (vocab/8 bytes per constrained row) go up and one token id per row comes back
        import numpy as np
        from ..ops.sampling import RowParams, pack_params, sample_rows
        if logits is None:
            logits = e.logits_rows(max(rows) + 1)
        if logits.dtype != torch.float32:
            logits = logits.float()
        picked = logits[torch.tensor(rows, device=logits.device)] if rows != list(range(len(rows))) else logits[:len(rows)]
        params, masks = [], []
        for r in reqs:
            s = r.sampling
            mask_row = -1
            m = r.constraint.mask() if r.constraint is not None else None
            if m is not None:
                mask_row = len(masks)
                masks.append(np.ascontiguousarray(m, dtype=np.uint32))
            params.append(RowParams(temperature=0.0 if s.greedy else s.temperature, top_k=s.top_k, top_p=s.top_p,
                                    min_p=s.min_p, seed=s.seed, position=getattr(r, "_emitted", 0), mask_row=mask_row))
        arena = None
        if masks:
            arena = torch.from_numpy(np.stack(masks).view(np.int32)).to(logits.device)
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
            self._release(a)
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

    def _spec_round(self, a: _Active):
        """One speculative round for the only active request: up to `width` tokens come back."""
        toks = self.spec.round_host()
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

    def _decode_round(self):
        e = self.e
        acts = self.active
        if len(acts) == 1 and acts[0].spec:
            return self._spec_round(acts[0])
        for a in acts:
            a.spec = False             # a request that shared a pass stays on plain decoding
        e.set_rows([a.last for a in acts], [a.pos for a in acts], [a.slot for a in acts])
        ep = self._engram_pass([a.last for a in acts], [a.slot for a in acts])
        e.forward_rows(len(acts))
        if ep is not None:
            self.engram.commit(ep)
        toks = self._select([a.req for a in acts], list(range(len(acts))))
        self.totals["rounds"] += 1
        keep = []
        for a, t in zip(acts, toks):
            a.pos += 1
            self.lanes.update(a.req.rid, a.req.max_tokens - a.emitted, a.pos)
            if self._emit(a, t):
                keep.append(a)
        self.active = keep
