#!/usr/bin/env python
"""Headline benchmark: C1 decode tokens/s of a DeepSeek-V4.1-Flash-shaped model with dSpark speculative decoding.

Config (BASELINE.json configs 2 and 5): full Flash architecture, random-init weights, routed experts FP8 E4M3 with
128x128 power-of-two block scales and 1x128 activation scales, dense/attention weights bf16, EP<N> experts and
TP<N> attention over N GPUs of one node, a 4096-token random-id prompt.  A dSpark-shaped one-stage drafter that
shares the target's embedding and head proposes 4 tokens per round; the target verifies the 5-row chunk; acceptance
follows the fixed schedule "3 of 4 drafts accepted" (random weights make real acceptance meaningless), so every
round emits 4 tokens.  Where the full model does not fit the N GPUs' memory the model is layer-truncated (the JSON
line says how many layers ran).  `--no-spec` times plain one-token-per-step greedy decoding instead.

  python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)
  python bench.py --impl reference ...                   (prints the reference arm's availability line)

Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events, max over ranks): K rounds replayed as CUDA
graphs with the accept rule and next-round inputs computed on the device.  `e2e` is the same metric through the
public SpecSession.round_host() call: per round the inputs come from pinned host memory and the emitted tokens
are read back to the host.
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


def reference_arm():
    why = ("pip install of /root/reference fails: \"Directory '/root/reference' is not installable. Neither 'setup.py' "
           "nor 'pyproject.toml' found.\" - the reference is a Rust/CMake engine whose kernels are AOT-exported for "
           "SM120/SM121 by absent submodules, and the image has no Rust toolchain")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


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


def prefill_bench(args, fabric, cfg, n_layers):
    """Prompt throughput: the whole prompt goes through DS41Engine.prefill in passes of --chunk rows (sorted expert
    path, sparse attention over the window and the selected compressed keys); a step is one whole prompt."""
    import torch
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    world, rank, dev = fabric.world, fabric.rank, fabric.device
    W, K = max(args.warmup, 3), args.steps
    t0 = time.time()
    weights = EngineWeights.random(cfg, rank, world, dev, seed=0, expert_dtype=args.expert_dtype)
    P = args.prompt
    if args.ced:
        # encoder / decoder-replay prompt passes: the boundary is the model's own (layer 20 of 40); a truncated stack
        # keeps the same half-and-half split if it still has no compressed source above it
        import dataclasses
        if not cfg.ced_on:
            cfg = dataclasses.replace(cfg, ced_boundary=args.ced_boundary or max(cfg.source_layers, default=0))
        if not cfg.ced_on:
            raise SystemExit("--ced: this layer count has no usable encoder/decoder boundary")
    eng = DS41Engine(cfg, weights, fabric, max_rows=args.chunk, slots=1, max_ctx=(P + 127) // 64 * 64)
    run_prompt = eng.prefill_ced if args.ced else eng.prefill
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(3, cfg.vocab - 600, (P,), generator=g).tolist()
    setup_s = time.time() - t0
    l0 = eng.launches
    for _ in range(W):
        run_prompt(0, prompt, chunk=args.chunk)
    per_prompt = (eng.launches - l0) // W
    eng.check_status("prefill warm-up")
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms = timed(fabric, torch, lambda: [run_prompt(0, prompt, chunk=args.chunk) for _ in range(K)])
    clocks = sampler.stop() if rank == 0 else {}
    eng.check_status("timed prefill")
    if args.breakdown:
        # every rank runs the pass (its kernels wait on the peers'); rank 0 prints its own event times, which include
        # the time its kernels spend waiting for slower peers
        fabric.barrier()
        eng.timeline = []
        run_prompt(0, prompt, chunk=args.chunk)
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
        run_prompt(0, prompt, chunk=args.chunk)
    torch.cuda.synchronize()
    e2e_s = fabric.all_reduce_max(time.perf_counter() - t1)
    if rank == 0:
        value = K * P / (ms / 1e3)
        chunks = (P + args.chunk - 1) // args.chunk
        line = {
            "metric": "prefill tok/s (one prompt, chunked passes)" if not args.ced else
                      f"prefill tok/s (one prompt, layers below {cfg.ced_boundary} over all tokens, layers from it "
                      f"upwards over the last {cfg.ced_replay})", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(value / BASELINE_PREFILL, 3),
            "dtype": "bf16 dense / fp8-e4m3 experts (fp32 accumulate)", "data": "synthetic",
            "config": {"model": f"DeepSeek-V4.1-Flash-shaped ({cfg.name})", "layers": n_layers, "layers_full_model": 40,
                       "global_batch": 1, "seq_len": P, "chunk_rows": args.chunk,
                       "parallelism": f"tp{world}+ep{world}",
                       "experts": {"mxfp8": "fp8 e4m3, 128x128 ue8m0 block scales, 1x128 activation scales",
                                   "mxfp4": "fp4 e2m1 weights, 1x32 ue8m0 scales (official layout), fp8 e4m3 activations "
                                            "with 1x128 scales", "bf16": "bf16",
                                   "nvfp4": "NVFP4 W4A4: e2m1 weights and activations, e4m3 scale per 16, fp32 scale per "
                                            "tensor"}[args.expert_dtype],
                       "l2": "no flush: every pass streams more weight bytes than the 126 MB L2",
                       "weights_gb_per_gpu": round(weights.nbytes() / 1e9, 2), "setup_s": round(setup_s, 1)},
            "clocks": clocks,
            "e2e": {"value": round(K * P / e2e_s, 1), "unit": "tok/s", "steps": K,
                    "h2d_bytes_per_step": 12 * P, "d2h_bytes_per_step": 4 * chunks},
            "gpu_launches": per_prompt * K, "impl": "ours",
        }
        print(json.dumps(line))
    fabric.barrier()
    return 0


def concurrent_bench(args, fabric, cfg, n_layers):
    """Concurrent greedy decode: C requests, one row each per step, all in one pass (paged KV, one slot per request).
    Prompts share their first half (the shared-prefix workload); this build recomputes the shared half per request."""
    import torch
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.runtime.session import DecodeSession
    world, rank, dev = fabric.world, fabric.rank, fabric.device
    C, P = args.concurrency, args.prompt
    W, K = max(args.warmup, 3), args.steps
    new_tokens = 2 * (W + K) + 8
    t0 = time.time()
    weights = EngineWeights.random(cfg, rank, world, dev, seed=0, expert_dtype=args.expert_dtype)
    eng = DS41Engine(cfg, weights, fabric, max_rows=max(C, args.chunk), slots=C,
                     max_ctx=(P + new_tokens + 127) // 64 * 64, kv_dtype=args.kv_dtype)
    g = torch.Generator().manual_seed(1234)
    shared = torch.randint(3, cfg.vocab - 600, (P // 2,), generator=g).tolist()
    first = []
    for s in range(C):
        own = torch.randint(3, cfg.vocab - 600, (P - P // 2,), generator=g).tolist()
        first.append(eng.prefill(s, shared + own, chunk=args.chunk))
    eng.check_status("prefill")
    setup_s = time.time() - t0
    sess = DecodeSession(eng, use_graphs=not args.no_graph)
    eng.set_rows(first, [P] * C, list(range(C)))
    sess.run_device_loop(C, W)
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms = timed(fabric, torch, lambda: sess.run_device_loop(C, K))
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
    fabric.barrier()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(K):
        toks = sess.step(toks, pos, slots)
        pos = [p + 1 for p in pos]
    torch.cuda.synchronize()
    e2e_s = fabric.all_reduce_max(time.perf_counter() - t1)
    eng.check_status("e2e decode")
    if rank == 0:
        value = C * K / (ms / 1e3)
        line = {
            "metric": f"decode tok/s C{C} (greedy, target-only)", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 dense / fp8-e4m3 experts (fp32 accumulate)", "data": "synthetic",
            "config": {"model": f"DeepSeek-V4.1-Flash-shaped ({cfg.name})", "layers": n_layers, "layers_full_model": 40,
                       "global_batch": C, "seq_len": P, "prompt_tokens": P, "parallelism": f"tp{world}+ep{world}",
                       "tokens_per_step": C, "kv_cache": f"paged, 64-token pages, {args.kv_dtype} rows",
                       "shared_prefix": "first half of every prompt identical; recomputed per request",
                       "experts": args.expert_dtype,
                       "l2": "no flush: every step streams more weight bytes than the 126 MB L2",
                       "weights_gb_per_gpu": round(weights.nbytes() / 1e9, 2),
                       "kv_gb_per_gpu": round(eng.cache.nbytes() / 1e9, 3), "setup_s": round(setup_s, 1)},
            "clocks": clocks,
            "e2e": {"value": round(C * K / e2e_s, 1), "unit": "tok/s", "steps": K,
                    "h2d_bytes_per_step": sess.h2d_bytes // max(K, 1), "d2h_bytes_per_step": sess.d2h_bytes // max(K, 1)},
            "gpu_launches": per_pass * K, "impl": "ours",
        }
        print(json.dumps(line))
    fabric.barrier()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64, help="timed rounds (speculative) or decode steps (--no-spec)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = fit to memory)")
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--model", default="flash", choices=["flash", "small", "tiny"])
    ap.add_argument("--expert-dtype", default="mxfp8", choices=["mxfp8", "mxfp4", "nvfp4", "bf16"])
    ap.add_argument("--prefill-chunk", type=int, default=32)
    ap.add_argument("--e2e-steps", type=int, default=0, help="rounds/steps of the host-loop measurement (0 = --steps)")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels eagerly (for per-kernel profiling)")
    ap.add_argument("--no-spec", action="store_true", help="plain greedy decoding, one token per step")
    ap.add_argument("--accept", type=int, default=3, help="drafts accepted per round in the fixed schedule")
    ap.add_argument("--draft-stages", type=int, default=1)
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"],
                    help="prefill: time whole-prompt passes in --chunk-row chunks (tok/s of prompt tokens)")
    ap.add_argument("--chunk", type=int, default=1024, help="rows per pass in --mode prefill")
    ap.add_argument("--concurrency", type=int, default=1, help="decode: number of concurrent requests (greedy, no drafter)")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"], help="latent KV rows in the cache")
    ap.add_argument("--ced", action="store_true",
                    help="prefill: the decoder layers run over the last 128 prompt tokens only (the reference's prompt "
                         "scheme); default is every layer over every token")
    ap.add_argument("--ced-boundary", type=int, default=0, help="first decoder layer for --ced on a truncated stack")
    ap.add_argument("--breakdown", action="store_true", help="prefill: per-kernel device time of one prompt (stderr)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()

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
        n_layers = args.layers or LAYERS_FOR_GPUS.get(world, 40)
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
    e2e_steps = args.e2e_steps or K
    total_new = (W + K + W + e2e_steps + 4) * per_round + 3 * width + 64
    max_ctx = (args.prompt + total_new + 4 * width + 127) // 64 * 64

    t0 = time.time()
    weights = EngineWeights.random(cfg, rank, world, dev, seed=0, expert_dtype=args.expert_dtype)
    eng = DS41Engine(cfg, weights, fabric, max_rows=max(args.prefill_chunk, width), slots=1, max_ctx=max_ctx,
                     kv_dtype=args.kv_dtype)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(3, cfg.vocab - 600, (args.prompt,), generator=g).tolist()
    assert eng.cache.ensure(0, max_ctx)
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
    run(W)
    per_pass_eager = (eng.launches + (drafter.eng.launches if drafter else 0) - l0) // W
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms = timed(fabric, torch, lambda: run(K))
    clocks = sampler.stop() if rank == 0 else {}
    eng.check_status("timed decode")
    if drafter:
        drafter.eng.check_status("timed decode (drafter)")
    if args.no_graph:
        per_pass = per_pass_eager
    else:
        per_pass = sess.launches_per_round if spec else sess.launches_per_graph.get((1, True), 0)
    launches = per_pass * K

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
        metric = (f"decode tok/s C1 (dSpark drafter, fixed acceptance {args.accept}/{width - 1})" if spec
                  else "decode tok/s C1 (greedy, target-only)")
        base = BASELINE_C1_DECODE if spec else BASELINE_TARGET_ONLY
        line = {
            "metric": metric, "value": round(value, 2), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(value / base, 3),
            "dtype": "bf16 dense / fp8-e4m3 experts (fp32 accumulate)", "data": "synthetic",
            "config": {"model": f"DeepSeek-V4.1-Flash-shaped ({cfg.name})", "layers": n_layers,
                       "layers_full_model": 40, "global_batch": 1, "seq_len": args.prompt,
                       "prompt_tokens": args.prompt, "parallelism": f"tp{world}+ep{world}",
                       "tokens_per_step": per_round,
                       "speculative": {"drafter_stages": args.draft_stages, "verify_rows": width,
                                       "accepted_per_round": args.accept} if spec else None,
                       "experts": {"mxfp8": "fp8 e4m3, 128x128 ue8m0 block scales, 1x128 activation scales",
                                   "mxfp4": "fp4 e2m1 weights, 1x32 ue8m0 scales (official layout), fp8 e4m3 activations "
                                            "with 1x128 scales", "bf16": "bf16",
                                   "nvfp4": "NVFP4 W4A4: e2m1 weights and activations, e4m3 scale per 16, fp32 scale per "
                                            "tensor"}[args.expert_dtype],
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
        print(json.dumps(line))
    fabric.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
