#!/usr/bin/env python
"""Benchmarks of the DeepSeek-V4.1-Flash-shaped engine: C1 decode with dSpark speculative decoding (the default and the
reference's headline), plain decode, concurrent decode and prompt throughput.

Default run: full Flash architecture, random-init weights, routed experts FP8 E4M3 with 128x128 power-of-two block
scales and 1x128 activation scales, dense / attention weights bf16, EP<N> experts and TP<N> attention over N GPUs of
one node, a 4096-token random-id prompt.  A dSpark-shaped drafter that shares the target's embedding and head proposes
4 tokens per round; the target verifies the 5-row chunk; acceptance follows the fixed schedule "3 of 4 drafts accepted"
(random weights make real acceptance meaningless), so every round emits 4 tokens.  Where the 40-layer model does not
fit the N GPUs' memory the stack is truncated: the metric names the layer count and `vs_baseline` (a ratio against
the reference's published 40-layer numbers) is then null; `vs_baseline_depth_scaled` is the same ratio with the
measured tokens/s multiplied by layers / 40.

Presets (`--config`): 2 = target-only C1 decode, 4096-token prompt, 512 greedy tokens; 3 = prompt throughput, 8 prompts
of 8192 tokens, router logits ~ N(0, 1) (`--skew`: two experts take about a quarter of the routed tokens); 4 = NVFP4
W4A4 experts, 64 concurrent requests, 2048-token prompts whose first 1024 tokens are one shared prefix restored from a
snapshot, 1024 output tokens, paged FP8 KV rows; 5 = speculative C1 decode over a 32 K-token context with a per-step
vocabulary mask on the target's choices.

  python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)
  python bench.py --impl reference ...                   (prints the reference arm's availability line)

Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events on the launching stream, barrier and
synchronize on both sides, max over ranks): K steps replayed as CUDA graphs with the accept rule and the next inputs
computed on the device.  The K-step measurement is repeated until about two seconds have been timed and the median
repeat is reported; clocks are sampled over the whole region.  `e2e` is the same metric through the public
SpecSession.round_host() / DecodeSession.step() call: per step the inputs come from pinned host memory and the
emitted tokens are read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

BASELINE_C1_DECODE = 146.12   # reference README.md:39 (1 RTX PRO 6000 + 4 DGX Spark, dSpark on)
BASELINE_TARGET_ONLY = 60.63  # reference README.md:109 (no drafts)
LAYERS_FOR_GPUS = {1: 10, 2: 22, 4: 40, 8: 40}


LAYERS_FULL = 40
MIN_TIMED_S = 2.0          # the K-step measurement is repeated until this much device time has been measured
MAX_REPEATS = 64


def reference_arm():
    why = ("pip install of the reference tree fails: \"Directory is not installable. Neither 'setup.py' nor "
           "'pyproject.toml' found.\" - the reference's serving engine is a Rust daemon (no Rust toolchain in the image) "
           "whose expert and projection GEMMs are AOT-exported for SM120/SM121 by absent submodules; its in-tree CUDA "
           "kernels do build (baseline/build_ref.py) and are timed one by one with "
           "`python -m ds41rt_b200.utils.kernel_case --impl reference`")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _provenance():
    """Digests of the sources this record was measured from (whole tree, kernel sources, host runtime, package), so a
    report can say which code a number belongs to.  Never fails the run: None when the tree cannot be read."""
    try:
        from ds41rt_b200.utils import source_manifest as sm
        d = sm.digests(sm.Path(__file__).resolve().parent)
        part = lambda prefix: sm.tree_digest({k: h for k, h in d.items() if k.startswith(prefix)})[:16]
        return {"tree": sm.tree_digest(d)[:16], "kernels": part("./csrc/kernels/"), "core": part("./csrc/core/"),
                "headers": part("./csrc/include/"), "python": part("./ds41rt_b200/")}
    except Exception:
        return None


def baseline_fields(value: float, base, n_layers: int) -> dict:
    """Ratios against a published 40-layer number: the plain ratio only for the full stack."""
    if base is None:
        return {"vs_baseline": None}
    full = n_layers >= LAYERS_FULL
    return {"vs_baseline": round(value / base, 3) if full else None,
            "vs_baseline_depth_scaled": round(value * min(n_layers, LAYERS_FULL) / LAYERS_FULL / base, 3),
            "baseline": {"value": base, "layers": LAYERS_FULL,
                         "note": "vs_baseline_depth_scaled = value x layers / 40 / baseline (per-layer cost taken as "
                                 "uniform; the head and the drafter are scaled down with it, so it understates)"}}


def layers_tag(n_layers: int) -> str:
    return "" if n_layers >= LAYERS_FULL else f", {n_layers} of {LAYERS_FULL} layers"


def timed_repeats(fabric, torch, run_k, est_ms: float, max_repeats: int = MAX_REPEATS):
    """Repeat the K-step measurement until about MIN_TIMED_S have been timed -> (median ms, all ms)."""
    reps = max(1, min(max_repeats, int(MIN_TIMED_S * 1e3 / max(est_ms, 1e-3)) + 1))
    times = [timed(fabric, torch, run_k) for _ in range(reps)]
    return statistics.median(times), times


class ClockSampler:
    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                 "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def timed(fabric, torch, fn):
    """Barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks -> ms."""
    fabric.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    fn()
    ev1.record()
    torch.cuda.synchronize()
    fabric.barrier()
    return fabric.all_reduce_max(ev0.elapsed_time(ev1))


BASELINE_PREFILL = 8355.0     # reference README.md:36 (best prefill, 2 RTX PRO 6000, v6 campaign)


def expert_note(dtype: str) -> str:
    return {"mxfp8": "fp8 e4m3, 128x128 ue8m0 block scales, 1x128 activation scales",
            "mxfp4": "fp4 e2m1 weights, 1x32 ue8m0 scales (official layout), fp8 e4m3 activations with 1x128 scales",
            "bf16": "bf16",
            "nvfp4": "NVFP4 W4A4: e2m1 weights and activations, e4m3 scale per 16, fp32 scale per tensor"}[dtype]


def skew_router(weights, cfg, hot: int = 2, bias: float = 0.94):
    """Push `hot` experts' selection bias up so that they are picked for most tokens (the skewed-load run)."""
    for lw in weights.layers:
        if lw is not None:
            lw.gate_bias[:hot] += bias


def prefill_bench(args, fabric, cfg, n_layers):
    """Prompt throughput: --prompts prompts, each run through DS41Engine.prefill in passes of --chunk rows (sorted expert
    path, sparse attention over the window and the selected compressed keys); a step is the whole batch of prompts."""
    import torch
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    world, rank, dev = fabric.world, fabric.rank, fabric.device
    W, K = max(args.warmup, 3), args.steps
    t0 = time.time()
    weights = EngineWeights.random(cfg, rank, world, dev, seed=0, expert_dtype=args.expert_dtype,
                                   router_std=args.router_std)
    if args.skew:
        skew_router(weights, cfg)
    P, NP = args.prompt, args.prompts
    if args.ced:
        # encoder / decoder-replay prompt passes: the boundary is the model's own (layer 20 of 40); a truncated stack
        # keeps the same half-and-half split if it still has no compressed source above it
        import dataclasses
        if not cfg.ced_on:
            cfg = dataclasses.replace(cfg, ced_boundary=args.ced_boundary or max(cfg.source_layers, default=0))
        if not cfg.ced_on:
            raise SystemExit("--ced: this layer count has no usable encoder/decoder boundary")
    eng = DS41Engine(cfg, weights, fabric, max_rows=args.chunk, slots=1, max_ctx=(P + 127) // 64 * 64,
                     long_pass=args.long_pass)
    run_prompt = eng.prefill_ced if args.ced else eng.prefill
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(3, cfg.vocab - 600, (P,), generator=g).tolist() for _ in range(NP)]
    setup_s = time.time() - t0

    def step():
        for pr in prompts:           # one request slot, reused: every prompt starts from an empty context
            run_prompt(0, pr, chunk=args.chunk)

    l0 = eng.launches
    est_ms = float("inf")
    for _ in range(W):
        torch.cuda.synchronize()
        tw = time.perf_counter()
        step()
        torch.cuda.synchronize()
        est_ms = min(est_ms, (time.perf_counter() - tw) * 1e3)
    per_step = (eng.launches - l0) // W
    eng.check_status("prefill warm-up")
    hot_share = None
    if args.skew:
        eng.debug = []
        run_prompt(0, prompts[0], chunk=args.chunk)
        ids = torch.cat([d["ids"].flatten() for d in eng.debug])
        hot_share = round(float((ids < 2).float().mean()), 4)
        eng.debug = None
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms, all_ms = timed_repeats(fabric, torch, lambda: [step() for _ in range(K)], est_ms * K)
    clocks = sampler.stop() if rank == 0 else {}
    eng.check_status("timed prefill")
    if args.breakdown:
        # every rank runs the pass (its kernels wait on the peers'); rank 0 prints its own event times, which include
        # the time its kernels spend waiting for slower peers
        fabric.barrier()
        eng.timeline = []
        run_prompt(0, prompts[0], chunk=args.chunk)
        torch.cuda.synchronize()
        acc = {}
        for tag, e0, e1 in eng.timeline:
            acc[tag] = acc.get(tag, 0.0) + e0.elapsed_time(e1)
        eng.timeline = None
        eng.check_status("breakdown pass")
        total = sum(acc.values())
        if rank == 0:
            for tag, v in sorted(acc.items(), key=lambda kv: -kv[1]):
                print(f"  {tag:24s} {v:9.3f} ms  {100 * v / total:5.1f}%", file=sys.stderr)
    # end to end: the same public call, wall clock around it (token ids go up and the next token comes back per call)
    fabric.barrier()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(K):
        step()
    torch.cuda.synchronize()
    e2e_s = fabric.all_reduce_max(time.perf_counter() - t1)
    if rank == 0:
        value = K * NP * P / (ms / 1e3)
        chunks = (P + args.chunk - 1) // args.chunk
        sp = eng._sp is not None
        scheme = "every layer over every token" if not args.ced else \
            f"layers below {cfg.ced_boundary} over all tokens, layers from it upwards over the last {cfg.ced_replay}"
        line = {
            "metric": f"prefill tok/s ({NP} prompt{'s' if NP > 1 else ''} of {P} tokens, {scheme}{layers_tag(n_layers)})",
            "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True,
            "scaling": "strong", **baseline_fields(value, BASELINE_PREFILL, n_layers),
            "repeats": len(all_ms), "timed_s": round(sum(all_ms) / 1e3, 3),
            "dtype": "bf16 dense / fp8-e4m3 experts (fp32 accumulate)", "data": "synthetic",
            "config": {"model": f"DeepSeek-V4.1-Flash-shaped ({cfg.name})", "layers": n_layers,
                       "layers_full_model": LAYERS_FULL, "global_batch": NP, "seq_len": P, "chunk_rows": args.chunk,
                       "parallelism": (f"sp{world} (row-sharded streams, unsharded dense weights) + ep{world}" if sp
                                       else f"tp{world}+ep{world}"),
                       "router": f"logits ~ N(0, {args.router_std}^2)" if args.router_std else "weights ~ N(0, 0.02^2)",
                       "skew": {"hot_experts": 2, "share_of_routed_tokens": hot_share} if args.skew else None,
                       "experts": expert_note(args.expert_dtype),
                       "l2": "no flush: every pass streams more weight bytes than the 126 MB L2",
                       "weights_gb_per_gpu": round(weights.nbytes() / 1e9, 2), "setup_s": round(setup_s, 1)},
            "clocks": clocks,
            "e2e": {"value": round(K * NP * P / e2e_s, 1), "unit": "tok/s", "steps": K,
                    "h2d_bytes_per_step": 12 * P * NP, "d2h_bytes_per_step": 4 * chunks * NP},
            "gpu_launches": per_step * K * len(all_ms), "impl": "ours",
        }
        line["source"] = _provenance()
        print(json.dumps(line))
    fabric.barrier()
    return 0


def concurrent_bench(args, fabric, cfg, n_layers):
    """Concurrent greedy decode: C requests, one row each per step, all in one pass (paged KV, one slot per request).
    The prompts share their first half: it is run once, snapshotted, and restored into every other slot (whole pages
    shared by reference, the cut page, window rings and pair carry copied); each request then runs only its own half."""
    import torch
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.runtime.session import DecodeSession
    world, rank, dev = fabric.world, fabric.rank, fabric.device
    C, P = args.concurrency, args.prompt
    W, K = max(args.warmup, 3), args.steps
    reps_max = max(1, min(MAX_REPEATS, 2048 // max(K, 1)))
    new_tokens = W + K * (reps_max + 1) + 16
    t0 = time.time()
    weights = EngineWeights.random(cfg, rank, world, dev, seed=0, expert_dtype=args.expert_dtype)
    max_ctx = (P + new_tokens + 127) // 64 * 64
    n_pages = C * ((max_ctx + 63) // 64) + 8
    eng = DS41Engine(cfg, weights, fabric, max_rows=max(C, args.chunk), slots=C, max_ctx=max_ctx, n_pages=n_pages,
                     kv_dtype=args.kv_dtype)
    g = torch.Generator().manual_seed(1234)
    n_shared = P // 2
    shared = torch.randint(3, cfg.vocab - 600, (n_shared,), generator=g).tolist()
    tp0 = time.time()
    eng.prefill(0, shared, chunk=args.chunk)
    snap = eng.cache.snapshot(0, n_shared)
    first = []
    for s in range(C):
        own = torch.randint(3, cfg.vocab - 600, (P - n_shared,), generator=g).tolist()
        if s > 0:
            assert eng.cache.restore(s, snap), "KV pool exhausted while restoring the shared prefix"
        first.append(eng.prefill(s, own, start=n_shared, chunk=args.chunk))
    torch.cuda.synchronize()
    prefill_s = time.time() - tp0
    eng.check_status("prefill")
    setup_s = time.time() - t0
    sess = DecodeSession(eng, use_graphs=not args.no_graph)
    eng.set_rows(first, [P] * C, list(range(C)))
    torch.cuda.synchronize()
    tw = time.perf_counter()
    sess.run_device_loop(C, W)
    torch.cuda.synchronize()
    est_ms = (time.perf_counter() - tw) * 1e3 / W
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms, all_ms = timed_repeats(fabric, torch, lambda: sess.run_device_loop(C, K), est_ms * K, reps_max)
    clocks = sampler.stop() if rank == 0 else {}
    eng.check_status("timed decode")
    per_pass = sess.launches_per_graph.get((C, True), 0) if not args.no_graph else 0
    # end to end: inputs from pinned host memory and the chosen tokens back to the host, every step
    toks = eng.in_tokens[:C].tolist()
    pos = eng.row_pos[:C].tolist()
    slots = list(range(C))
    for _ in range(3):
        toks = sess.step(toks, pos, slots)
        pos = [p + 1 for p in pos]
    sess.h2d_bytes = sess.d2h_bytes = 0
    e2e_steps = min(K, 64)
    fabric.barrier()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(e2e_steps):
        toks = sess.step(toks, pos, slots)
        pos = [p + 1 for p in pos]
    torch.cuda.synchronize()
    e2e_s = fabric.all_reduce_max(time.perf_counter() - t1)
    eng.check_status("e2e decode")
    if rank == 0:
        value = C * K / (ms / 1e3)
        line = {
            "metric": f"decode tok/s C{C} (greedy, target-only{layers_tag(n_layers)})", "value": round(value, 1),
            "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "repeats": len(all_ms), "timed_s": round(sum(all_ms) / 1e3, 3),
            "dtype": "bf16 dense / " + args.expert_dtype + " experts (fp32 accumulate)", "data": "synthetic",
            "config": {"model": f"DeepSeek-V4.1-Flash-shaped ({cfg.name})", "layers": n_layers,
                       "layers_full_model": LAYERS_FULL,
                       "global_batch": C, "seq_len": P, "prompt_tokens": P, "parallelism": f"tp{world}+ep{world}",
                       "tokens_per_step": C, "kv_cache": f"paged, 64-token pages, {args.kv_dtype} rows",
                       "shared_prefix": {"tokens": n_shared, "reuse": "run once, snapshot restored into every other slot "
                                         "(pages shared by reference)", "pages_shared": len(snap.pages),
                                         "prompt_phase_s": round(prefill_s, 2)},
                       "experts": expert_note(args.expert_dtype),
                       "reference_concurrency_cap": 16,
                       "l2": "no flush: every step streams more weight bytes than the 126 MB L2",
                       "weights_gb_per_gpu": round(weights.nbytes() / 1e9, 2),
                       "kv_gb_per_gpu": round(eng.cache.nbytes() / 1e9, 3), "setup_s": round(setup_s, 1)},
            "clocks": clocks,
            "e2e": {"value": round(C * e2e_steps / e2e_s, 1), "unit": "tok/s", "steps": e2e_steps,
                    "h2d_bytes_per_step": sess.h2d_bytes // max(e2e_steps, 1),
                    "d2h_bytes_per_step": sess.d2h_bytes // max(e2e_steps, 1)},
            "gpu_launches": per_pass * K * len(all_ms), "impl": "ours",
        }
        line["source"] = _provenance()
        print(json.dumps(line))
    fabric.barrier()
    return 0


PRESETS = {
    2: dict(no_spec=True, prompt=4096, steps=512),
    3: dict(mode="prefill", prompts=8, prompt=8192, chunk=8192, router_std=1.0, steps=2),
    4: dict(concurrency=64, prompt=2048, steps=1024, expert_dtype="nvfp4", kv_dtype="fp8"),
    5: dict(prompt=32768, prefill_chunk=2048, mask=True),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed rounds (speculative) or decode steps / prompt batches")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", type=int, default=0, choices=[0, 2, 3, 4, 5],
                    help="preset of one of the named benchmark configurations (explicit flags still win)")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = fit to memory)")
    ap.add_argument("--prompt", type=int, default=None)
    ap.add_argument("--prompts", type=int, default=None, help="prefill: prompts per step")
    ap.add_argument("--model", default="flash", choices=["flash", "small", "tiny"])
    ap.add_argument("--expert-dtype", default=None, choices=["mxfp8", "mxfp4", "nvfp4", "bf16"])
    ap.add_argument("--prefill-chunk", type=int, default=None)
    ap.add_argument("--e2e-steps", type=int, default=0, help="rounds/steps of the host-loop measurement (0 = --steps)")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels eagerly (for per-kernel profiling)")
    ap.add_argument("--no-spec", action="store_true", default=None, help="plain greedy decoding, one token per step")
    ap.add_argument("--accept", type=int, default=3, help="drafts accepted per round in the fixed schedule")
    ap.add_argument("--draft-stages", type=int, default=1)
    ap.add_argument("--mode", default=None, choices=["decode", "prefill"],
                    help="prefill: time whole-prompt passes in --chunk-row chunks (tok/s of prompt tokens)")
    ap.add_argument("--chunk", type=int, default=None, help="rows per pass in --mode prefill")
    ap.add_argument("--concurrency", type=int, default=None, help="decode: number of concurrent requests (greedy, no drafter)")
    ap.add_argument("--kv-dtype", default=None, choices=["bf16", "fp8", "fp4"], help="latent KV rows in the cache")
    ap.add_argument("--router-std", type=float, default=None, help="standard deviation of the router logits (prefill)")
    ap.add_argument("--skew", action="store_true", help="prefill: two experts take about a quarter of the routed tokens")
    ap.add_argument("--mask", action="store_true", default=None,
                    help="speculative decode: a vocabulary allow-mask (synthetic, 1 token in 4 allowed) on every "
                         "verification row, applied in the target's selection kernel")
    ap.add_argument("--long-pass", default="auto", choices=["auto", "sp", "replicated"],
                    help="multi-GPU long passes: row-sharded (sp) or replicated rows with sharded heads")
    ap.add_argument("--ced", action="store_true",
                    help="prefill: the decoder layers run over the last 128 prompt tokens only (the reference's prompt "
                         "scheme); default is every layer over every token")
    ap.add_argument("--ced-boundary", type=int, default=0, help="first decoder layer for --ced on a truncated stack")
    ap.add_argument("--breakdown", action="store_true", help="prefill: per-kernel device time of one prompt (stderr)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    defaults = dict(steps=64, prompt=4096, prompts=1, expert_dtype="mxfp8", prefill_chunk=32, no_spec=False,
                    mode="decode", chunk=1024, concurrency=1, kv_dtype="bf16", router_std=None, mask=False)
    defaults.update(PRESETS.get(args.config, {}))
    for key, val in defaults.items():
        if getattr(args, key) is None:
            setattr(args, key, val)

    import dataclasses

    import torch
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.dspark import DSparkDrafter
    from ds41rt_b200.parallel.fabric import Fabric
    from ds41rt_b200.runtime.session import DecodeSession
    from ds41rt_b200.runtime.speculative import SpecSession

    fabric = Fabric.create()
    world, rank = fabric.world, fabric.rank
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run",
                  file=sys.stderr)
        return 2
    dev = fabric.device
    if args.model == "flash":
        n_layers = args.layers or LAYERS_FOR_GPUS.get(world, LAYERS_FULL)
        cfg = ModelConfig.flash(n_layers)
    else:
        cfg = getattr(ModelConfig, args.model)()
        n_layers = cfg.n_layers
    if args.mode == "prefill":
        return prefill_bench(args, fabric, cfg, n_layers)
    if args.concurrency > 1:
        return concurrent_bench(args, fabric, cfg, n_layers)
    spec = not args.no_spec
    if spec:
        cfg.dspark = dataclasses.replace(cfg.dspark, stages=args.draft_stages)
    width = cfg.dspark.block_size if spec else 1
    per_round = args.accept + 1 if spec else 1
    W, K = max(args.warmup, 3), args.steps
    e2e_steps = args.e2e_steps or min(K, 256)
    reps_max = max(1, min(MAX_REPEATS, 2048 // max(K, 1)))
    total_new = (2 * W + K * (reps_max + 1) + e2e_steps + 4) * per_round + 3 * width + 64
    max_ctx = (args.prompt + total_new + 4 * width + 127) // 64 * 64

    t0 = time.time()
    weights = EngineWeights.random(cfg, rank, world, dev, seed=0, expert_dtype=args.expert_dtype)
    eng = DS41Engine(cfg, weights, fabric, max_rows=max(args.prefill_chunk, width), slots=1, max_ctx=max_ctx,
                     kv_dtype=args.kv_dtype)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(3, cfg.vocab - 600, (args.prompt,), generator=g).tolist()
    assert eng.cache.ensure(0, max_ctx)
    if args.mask:
        # one allow-mask row per verification row: a fixed pseudo-random quarter of the vocabulary (the stand-in for
        # the per-step masks a grammar matcher produces; real constraints come from runtime/grammar.py)
        words = (cfg.vocab + 31) // 32
        gm = torch.Generator().manual_seed(99)
        m = torch.randint(0, 2 ** 31 - 1, (width, words), generator=gm, dtype=torch.int64) & \
            torch.randint(0, 2 ** 31 - 1, (width, words), generator=gm, dtype=torch.int64)
        eng.head_mask = m.to(torch.int32).to(dev)
    drafter = None
    if spec:
        drafter = DSparkDrafter(cfg, eng, weights=None, seed=0, expert_dtype=args.expert_dtype)
        sess = SpecSession(eng, drafter, forced_accept=args.accept, use_graphs=not args.no_graph)
        sess.start(0, prompt, total_new, chunk=args.prefill_chunk)
    else:
        sess = DecodeSession(eng, use_graphs=not args.no_graph)
        first = eng.prefill(0, prompt, chunk=args.prefill_chunk)
        eng.set_rows([first], [args.prompt], [0])
    torch.cuda.synchronize()
    eng.check_status("prefill")
    setup_s = time.time() - t0

    def run(n):
        if spec:
            for _ in range(n):
                sess.round()
        else:
            sess.run_device_loop(1, n)

    # ---------------- device-timed: K graph replays, accept rule / token feedback on the device
    l0 = eng.launches + (drafter.eng.launches if drafter else 0)
    run(3)                                  # graph capture and first replays
    torch.cuda.synchronize()
    tw = time.perf_counter()
    run(W)
    torch.cuda.synchronize()
    est_ms = (time.perf_counter() - tw) * 1e3 / W
    per_pass_eager = (eng.launches + (drafter.eng.launches if drafter else 0) - l0) // (W + 3)
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms, all_ms = timed_repeats(fabric, torch, lambda: run(K), est_ms * K, reps_max)
    clocks = sampler.stop() if rank == 0 else {}
    eng.check_status("timed decode")
    if drafter:
        drafter.eng.check_status("timed decode (drafter)")
    if args.no_graph:
        per_pass = per_pass_eager
    else:
        per_pass = sess.launches_per_round if spec else sess.launches_per_graph.get((1, True), 0)
    launches = per_pass * K * len(all_ms)

    # ---------------- end to end through the public API: pinned H2D in, D2H out, every round/step
    if spec:
        for _ in range(W):
            sess.round_host(feed_inputs=True)
        sess.h2d_bytes = sess.d2h_bytes = 0
        fabric.barrier()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        emitted = 0
        for _ in range(e2e_steps):
            emitted += len(sess.round_host(feed_inputs=True))
        torch.cuda.synchronize()
        e2e_s = fabric.all_reduce_max(time.perf_counter() - t1)
        e2e_tokens = emitted
    else:
        pos = int(eng.row_pos[0].item())
        tok = int(eng.in_tokens[0].item())
        for _ in range(W):
            tok = sess.step([tok], [pos], [0])[0]
            pos += 1
        sess.h2d_bytes = sess.d2h_bytes = 0
        fabric.barrier()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(e2e_steps):
            tok = sess.step([tok], [pos], [0])[0]
            pos += 1
        torch.cuda.synchronize()
        e2e_s = fabric.all_reduce_max(time.perf_counter() - t1)
        e2e_tokens = e2e_steps
    eng.check_status("e2e decode")

    if rank == 0:
        value = K * per_round / (ms / 1e3)
        tag = layers_tag(n_layers) + (", vocabulary mask on every verification row" if args.mask else "")
        metric = (f"decode tok/s C1 (dSpark drafter, fixed acceptance {args.accept}/{width - 1}{tag})" if spec
                  else f"decode tok/s C1 (greedy, target-only{tag})")
        base = BASELINE_C1_DECODE if spec else BASELINE_TARGET_ONLY
        line = {
            "metric": metric, "value": round(value, 2), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "strong", **baseline_fields(value, base, n_layers),
            "repeats": len(all_ms), "timed_s": round(sum(all_ms) / 1e3, 3),
            "dtype": "bf16 dense / fp8-e4m3 experts (fp32 accumulate)", "data": "synthetic",
            "config": {"model": f"DeepSeek-V4.1-Flash-shaped ({cfg.name})", "layers": n_layers,
                       "layers_full_model": LAYERS_FULL, "global_batch": 1, "seq_len": args.prompt,
                       "prompt_tokens": args.prompt, "context_at_end": int(eng.row_pos[0].item()),
                       "parallelism": f"tp{world}+ep{world}", "tokens_per_step": per_round,
                       "speculative": {"drafter_stages": args.draft_stages, "verify_rows": width,
                                       "accepted_per_round": args.accept} if spec else None,
                       "experts": expert_note(args.expert_dtype),
                       "l2": "no flush: every step streams more weight bytes than the 126 MB L2",
                       "weights_gb_per_gpu": round(weights.nbytes() / 1e9, 2),
                       "kv_gb_per_gpu": round(eng.cache.nbytes() / 1e9, 3), "setup_s": round(setup_s, 1)},
            "clocks": clocks,
            "e2e": {"value": round(e2e_tokens / e2e_s, 2), "unit": "tok/s", "steps": e2e_steps,
                    "h2d_bytes_per_step": sess.h2d_bytes // max(e2e_steps, 1),
                    "d2h_bytes_per_step": sess.d2h_bytes // max(e2e_steps, 1)},
            "gpu_launches": launches,
            "impl": "ours",
        }
        line["source"] = _provenance()
        print(json.dumps(line))
    fabric.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
