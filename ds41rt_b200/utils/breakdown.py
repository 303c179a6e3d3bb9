"""Per-kernel time breakdown of one decode step, measured inside CUDA graphs.

For every kernel tag of the engine's launch sequence a graph holding ONLY that tag's launches (all layers) is
captured and replayed; CUDA events around the replays give the warm, launch-overhead-free device time of that
kernel class.  `python -m ds41rt_b200.utils.breakdown --layers 11` prints a table (and JSON with --json).
`--spec` breaks down a whole speculative round instead (draft pass of the dSpark drafter, verification pass of `width`
rows, ring feed, accept rule; fixed acceptance 3 of 4): drafter kernels are listed with a `draft:` prefix.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..config import ModelConfig
from ..models.ds41 import DS41Engine, EngineWeights
from ..parallel.fabric import Fabric


def time_graph(fn, reps: int = 20) -> float:
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3     # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=640)
    ap.add_argument("--model", default="flash")
    ap.add_argument("--expert-dtype", default="mxfp8")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--spec", action="store_true", help="break down one speculative round (drafter + verification)")
    args = ap.parse_args()
    fabric = Fabric.create()
    cfg = ModelConfig.flash(args.layers) if args.model == "flash" else getattr(ModelConfig, args.model)()
    w = EngineWeights.random(cfg, fabric.rank, fabric.world, fabric.device, expert_dtype=args.expert_dtype)
    eng = DS41Engine(cfg, w, fabric, max_rows=max(64, args.rows), slots=1,
                     max_ctx=args.prompt + (1280 if args.spec else 256))
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(3, cfg.vocab - 600, (args.prompt,), generator=g).tolist()
    if args.spec:
        return spec_round_breakdown(args, fabric, cfg, eng, prompt)
    eng.cache.ensure(0, args.prompt + 128)
    nxt = eng.prefill(0, prompt)
    R = args.rows
    eng.set_rows([nxt] * R, list(range(args.prompt, args.prompt + R)), [0] * R)
    # discover tags
    tags = []
    orig = eng._run

    def spy(tag, fn, *a, **kw):
        if tag not in tags:
            tags.append(tag)
        return orig(tag, fn, *a, **kw)
    eng._run = spy
    before = eng.launches
    eng.forward_rows(R)
    total_launches = eng.launches - before
    eng._run = orig
    torch.cuda.synchronize()
    eng.check_status("breakdown warm-up")
    full = time_graph(lambda: eng.forward_rows(R))
    rows = []
    for t in tags:
        eng.only = {t}
        b0 = eng.launches
        eng.forward_rows(R)
        n = eng.launches - b0
        us = time_graph(lambda: eng.forward_rows(R))
        rows.append((t, n, us))
    eng.only = None
    eng.check_status("breakdown")
    if fabric.rank == 0:
        s = sum(r[2] for r in rows)
        if args.json:
            print(json.dumps({"step_us": full, "launches": total_launches, "sum_us": s,
                              "kernels": {t: {"launches": n, "us": us} for t, n, us in rows}}))
        else:
            print(f"full step: {full:.1f} us in {total_launches} launches; sum of isolated classes {s:.1f} us")
            for t, n, us in sorted(rows, key=lambda r: -r[2]):
                print(f"  {t:20s} x{n:3d}  {us:9.1f} us  ({us / max(n, 1):6.2f} us each)  {100 * us / s:5.1f}%")
    fabric.barrier()


def spec_round_breakdown(args, fabric, cfg, eng, prompt):
    from ..models.dspark import DSparkDrafter
    from ..runtime.speculative import SpecSession
    drafter = DSparkDrafter(cfg, eng, weights=None, seed=0, expert_dtype=args.expert_dtype)
    sess = SpecSession(eng, drafter, forced_accept=drafter.width - 2, use_graphs=False)
    sess.start(0, prompt, 1024)        # room for the rounds that the timing loops replay
    engines = (("", eng), ("draft:", drafter.eng))
    tags = []
    origs = [e._run for _, e in engines]

    def spy(prefix, orig):
        def run(tag, fn, *a, **kw):
            if prefix + tag not in tags:
                tags.append(prefix + tag)
            return orig(tag, fn, *a, **kw)
        return run
    for (prefix, e), orig in zip(engines, origs):
        e._run = spy(prefix, orig)
    before = eng.launches + drafter.eng.launches
    sess._enqueue_round()
    total_launches = eng.launches + drafter.eng.launches - before
    for (_, e), orig in zip(engines, origs):
        e._run = orig
    torch.cuda.synchronize()
    eng.check_status("breakdown warm-up")
    full = time_graph(sess._enqueue_round)
    rows = []
    for t in tags:
        for prefix, e in engines:
            mine = t.startswith("draft:") == (prefix == "draft:")
            e.only = {t[len(prefix):]} if mine else {"-"}
        b0 = eng.launches + drafter.eng.launches
        sess._enqueue_round()
        n = eng.launches + drafter.eng.launches - b0
        rows.append((t, n, time_graph(sess._enqueue_round)))
    for _, e in engines:
        e.only = None
    eng.check_status("breakdown")
    drafter.eng.check_status("breakdown (drafter)")
    if fabric.rank == 0:
        s = sum(r[2] for r in rows)
        if args.json:
            print(json.dumps({"round_us": full, "launches": total_launches, "sum_us": s,
                              "kernels": {t: {"launches": n, "us": us} for t, n, us in rows}}))
        else:
            print(f"speculative round: {full:.1f} us in {total_launches} launches; sum of isolated classes {s:.1f} us")
            for t, n, us in sorted(rows, key=lambda r: -r[2]):
                print(f"  {t:26s} x{n:3d}  {us:9.1f} us  ({us / max(n, 1):6.2f} us each)  {100 * us / s:5.1f}%")
    fabric.barrier()


if __name__ == "__main__":
    main()
