"""Prefill matrix through the serving backend: time to first token for a suffix on top of a cold or retained base.

    python -m ds41rt_b200.utils.prefill_matrix --model flash --layers 10 --bases 0,8192,32768 --suffixes 1024,4096,8192

For every base length B (tokens already seen by the server) and suffix length S the tool sends a prompt of B + S tokens
whose first B tokens repeat an earlier prompt, so that the server restores the base from its prompt snapshot and runs
only the suffix ("retained" rows), and the same prompt against a server without any snapshot ("cold" rows: B + S tokens
are computed).  Requests go through `serving.engine.NativeBackend` exactly as the HTTP layer submits them (admission,
page leases, prefix restore, chunked prompt passes interleaved by the scheduler, first-token selection); the clock
runs from `submit` to the first token event.  One JSON line per row and a closing summary line.
Counterpart of the reference's release prefill matrix (scripts/bench-ds41-release-prefill-matrix.py: bases x suffixes,
cold and retained).
"""
from __future__ import annotations

import argparse
import json
import time
from typing import List, Optional


def first_token_seconds(backend, prompt: List[int], timeout: float = 600.0):
    """Submit one greedy request of one token -> (seconds to its first token, prompt_cache_hit_tokens)."""
    from ..serving.engine import GenRequest
    from ..serving.protocol import Sampling
    r = GenRequest(prompt_ids=prompt, max_tokens=1, sampling=Sampling(temperature=0.0))
    t0 = time.perf_counter()
    backend.submit(r)
    hit, first = 0, None
    while True:
        ev = r.events.get(timeout=timeout)
        if ev.kind == "ready":
            hit = (ev.usage or {}).get("prompt_cache_hit_tokens", 0)
        elif ev.kind == "tokens" and first is None:
            first = time.perf_counter() - t0
        elif ev.kind == "finish":
            return (first if first is not None else time.perf_counter() - t0), hit
        elif ev.kind == "error":
            raise RuntimeError(ev.message)


def run_matrix(backend, vocab: int, bases: List[int], suffixes: List[int], seed: int = 0, warm: bool = True,
               emit=None) -> List[dict]:
    """Rows {"base", "suffix", "mode", "seconds", "computed_tokens", "tok_per_s", "cache_hit_tokens"}."""
    import torch
    g = torch.Generator().manual_seed(seed)
    rand = lambda n: torch.randint(3, max(4, vocab - 8), (n,), generator=g).tolist()
    rows = []

    def drop_snapshots():
        for sid in list(backend.snapshots):
            backend._drop_snapshot(sid)

    def record(base, suffix, mode, seconds, hit):
        computed = base + suffix - hit
        row = {"base": base, "suffix": suffix, "mode": mode, "seconds": round(seconds, 4), "computed_tokens": computed,
               "tok_per_s": round(computed / seconds, 1) if seconds > 0 else 0.0, "cache_hit_tokens": hit}
        rows.append(row)
        if emit:
            emit(row)

    if warm:                                              # kernels, graphs and allocator warm before the first clock
        first_token_seconds(backend, rand(min(max(suffixes), 512)))
    for base in bases:
        base_prompt = rand(base) if base else []
        for suffix in suffixes:
            prompt = base_prompt + rand(suffix)
            _idle(backend)
            drop_snapshots()
            sec, hit = first_token_seconds(backend, prompt)
            record(base, suffix, "cold", sec, hit)
            if base:
                _idle(backend)
                drop_snapshots()
                first_token_seconds(backend, base_prompt)  # the earlier turn: leaves the base's snapshot behind
                _idle(backend)
                sec, hit = first_token_seconds(backend, prompt)
                record(base, suffix, "retained", sec, hit)
    return rows


def _idle(backend, timeout: float = 60.0):
    """Wait until the worker has retired everything (snapshots are touched only by the worker between requests)."""
    t0 = time.time()
    while (backend.active or backend.prefilling is not None or backend.q.qsize()) and time.time() - t0 < timeout:
        time.sleep(0.002)


def main(argv: Optional[List[str]] = None) -> int:
    import torch
    from ..config import ModelConfig
    from ..models.ds41 import DS41Engine, EngineWeights
    from ..serving.engine import NativeBackend
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="flash", choices=["flash", "small", "tiny"])
    ap.add_argument("--layers", type=int, default=10)
    ap.add_argument("--expert-dtype", default="mxfp8")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"])
    ap.add_argument("--bases", default="0,8192,32768")
    ap.add_argument("--suffixes", default="1024,4096,8192")
    ap.add_argument("--prefill-chunk", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    bases = [int(x) for x in args.bases.split(",") if x]
    suffixes = [int(x) for x in args.suffixes.split(",") if x]
    dev = torch.device("cuda", 0)
    cfg = ModelConfig.flash(args.layers) if args.model == "flash" else getattr(ModelConfig, args.model)()
    weights = EngineWeights.random(cfg, 0, 1, dev, seed=args.seed,
                                   expert_dtype=args.expert_dtype if args.model == "flash" else "bf16")
    chunk = min(args.prefill_chunk, max(suffixes))
    eng = DS41Engine(cfg, weights, max_rows=max(64, chunk), slots=2, max_ctx=max(bases) + max(suffixes) + 64,
                     kv_dtype=args.kv_dtype)
    backend = NativeBackend(eng, eos=-1, concurrency=1, prefill_chunk=chunk, prompt_snapshots=4, turn_snapshots=2)
    try:
        rows = run_matrix(backend, cfg.vocab, bases, suffixes, args.seed, emit=lambda r: print(json.dumps(r), flush=True))
        st = backend.stats()["totals"]
        print(json.dumps({"summary": True, "model": cfg.name, "layers": cfg.n_layers, "expert_dtype": args.expert_dtype,
                          "kv_dtype": args.kv_dtype, "prefill_chunk": chunk, "rows": len(rows),
                          "ced_prefills": st.get("ced_prefills", 0), "prefill_passes": st.get("prefill_passes", 0),
                          "prompt_cache_hit_tokens": st.get("prompt_cache_hit_tokens", 0)}))
    finally:
        backend.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
