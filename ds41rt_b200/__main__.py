"""Command line: `python -m ds41rt_b200 <command>`.

  build                      compile the kernel and host-runtime libraries in-tree
  serve  [--model ...]       OpenAI-compatible HTTP server over the native engine; under torch.distributed.run rank 0
                             serves and the other ranks mirror its engine calls (tensor + expert parallel)
  info                       print the model configuration and the per-rank memory plan

The reference's counterparts are its run.sh / build.sh launchers and the `v41-native-serve` daemon command
(rust/crates/ds41rt-daemon/src/v41_native_serve.rs, rust/crates/ds41rt-daemon/src/cli.rs).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _config(args):
    from .config import ModelConfig
    if args.config:
        with open(args.config) as f:
            return ModelConfig.from_official_json(json.load(f))
    if args.model == "flash":
        return ModelConfig.flash(args.layers or 4)
    return ModelConfig.small() if args.model == "small" else ModelConfig.tiny()


def cmd_build(args) -> int:
    from . import build
    build.build_kernels()
    build.build_core()
    print("built", flush=True)
    return 0


def cmd_info(args) -> int:
    from .loader.catalog import expected_tensors
    cfg = _config(args)
    n = len(expected_tensors(cfg)) if args.model == "flash" and not args.layers else None
    expert = 3 * cfg.hidden * cfg.inter
    print(json.dumps({"model": cfg.name, "layers": cfg.n_layers, "hidden": cfg.hidden, "experts": cfg.n_experts,
                      "topk": cfg.topk, "vocab": cfg.vocab, "checkpoint_tensors": n,
                      "expert_bytes_fp8": expert, "experts_gb_per_layer_fp8": round(expert * cfg.n_experts / 2 ** 30, 2)}))
    return 0


def _attach_engram(args, cfg, eng, dev):
    """Every rank: give the engine its Engram layers (checkpoint weights, or random ones for a random-init model).
    Returns the decoder layers that have one, in hash-family order."""
    if cfg.engram is None or not (args.engram_table or args.engram_random_rows):
        return []
    import torch
    from .models.engram import EngramLayer, init_engram_weights
    layers = [l for l in cfg.engram.layers if l < eng.n_layers]
    for i, l in enumerate(layers):
        if args.checkpoint:
            from .loader.official import load_engram_layer
            mod = load_engram_layer(args.checkpoint, cfg, l, dev)
        else:
            wkv, q_w, k_w = init_engram_weights(cfg.hidden, seed=args.seed + 31 * i, std=0.002)
            bf = lambda t: t.to(device=dev, dtype=torch.bfloat16)
            mod = EngramLayer(bf(wkv), bf(q_w), bf(k_w), cfg.hidden)
        eng.attach_engram(l, mod)
    return layers


def _engram_pipeline(args, cfg, eng, layers, tokenizer):
    """Rank 0: the tables and the gather threads behind the engine's Engram layers."""
    if not layers:
        return None
    import tempfile
    from .models.engram import random_table_rows
    from .runtime.engram import EngramPipeline, compressed_token_ids
    from .runtime.engram_io import EngramTable
    tables = []
    for i, l in enumerate(layers):
        if args.engram_table:
            n_rows = cfg.engram.num_embeddings[cfg.engram.layers.index(l)]
            tables.append(EngramTable(args.engram_table[i], n_rows, 264))
        else:                                        # a small random table, row ids folded into it
            path = os.path.join(tempfile.mkdtemp(prefix="ds41-engram-"), f"layer{l}.bin")
            random_table_rows(args.engram_random_rows, seed=args.seed + i).numpy().tofile(path)
            tables.append(EngramTable(path, args.engram_random_rows, 264))
    return EngramPipeline(layers, tables, token_map=compressed_token_ids(tokenizer.token_bytes()),
                          pad_id=cfg.engram.pad_token_id, max_rows=eng.max_rows, fold=not args.engram_table)


def cmd_serve(args) -> int:
    import torch
    from .models.ds41 import DS41Engine, EngineWeights
    from .serving.engine import NativeBackend
    from .serving.http import ApiServer
    from .serving.tokenizer import ByteTokenizer, HFTokenizer
    if not torch.cuda.is_available():
        print("serve needs a CUDA device", file=sys.stderr)
        return 2
    from .parallel.fabric import Fabric
    from .serving.distributed import LeaderEngine, follower_loop, make_control_group
    cfg = _config(args)
    fabric = Fabric.create() if "WORLD_SIZE" in os.environ else Fabric.single(torch.device("cuda", args.device))
    rank, world, dev = fabric.rank, fabric.world, fabric.device
    ctl = make_control_group(fabric)
    tk = HFTokenizer(args.tokenizer) if args.tokenizer else ByteTokenizer(vocab_size=cfg.vocab)
    t0 = time.time()
    if args.checkpoint:
        from .loader.official import load_engine_weights
        weights = load_engine_weights(args.checkpoint, cfg, rank, world, dev, expert_dtype=args.expert_dtype)
    else:
        weights = EngineWeights.random(cfg, rank, world, dev, seed=args.seed, expert_dtype=args.expert_dtype)
    eng = DS41Engine(cfg, weights, fabric, max_rows=max(8, args.concurrency), slots=args.concurrency,
                     max_ctx=args.max_context, kv_dtype=args.kv_dtype)
    engram_layers = _attach_engram(args, cfg, eng, dev)
    if rank != 0:
        # every other rank mirrors the leader's engine calls until it is told to stop
        follower_loop(eng, ctl, on_error=lambda e: print(f"rank {rank}: {e}", file=sys.stderr, flush=True))
        return 0
    lead = LeaderEngine(eng, ctl)
    drafter = None
    if args.speculative:
        if world > 1:
            print("--speculative serves from one rank only in this build; ignoring it", file=sys.stderr)
        else:
            from .models.dspark import DSparkDrafter
            drafter = DSparkDrafter(cfg, eng, weights=None, seed=args.seed, expert_dtype=args.expert_dtype)
    backend = NativeBackend(lead if world > 1 else eng, eos=tk.eos, concurrency=args.concurrency,
                            queue_depth=args.queue_depth, drafter=drafter,
                            engram=_engram_pipeline(args, cfg, eng, engram_layers, tk))
    srv = ApiServer(backend, tk, host=args.host, port=args.port, queue_depth=args.queue_depth, waiters=args.waiters,
                    max_context=args.max_context).start()
    print(json.dumps({"listening": f"http://{args.host}:{srv.port}", "model": cfg.name, "ranks": world,
                      "setup_s": round(time.time() - t0, 1)}), flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        pass
    finally:
        srv.stop()
        backend.close()
        lead.stop_followers()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ds41rt_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def model_args(p):
        p.add_argument("--model", default="tiny", choices=["tiny", "small", "flash"])
        p.add_argument("--layers", type=int, default=0, help="flash: number of layers to instantiate")
        p.add_argument("--config", default="", help="official config.json (overrides --model)")

    sub.add_parser("build")
    pi = sub.add_parser("info")
    model_args(pi)
    ps = sub.add_parser("serve")
    model_args(ps)
    ps.add_argument("--checkpoint", default="", help="directory with model.safetensors.index.json (official layout)")
    ps.add_argument("--tokenizer", default="", help="tokenizer.json; default: byte-level tokenizer")
    ps.add_argument("--expert-dtype", default="mxfp8", choices=["mxfp8", "mxfp4", "nvfp4", "bf16"])
    ps.add_argument("--host", default="127.0.0.1")
    ps.add_argument("--port", type=int, default=8000)
    ps.add_argument("--device", type=int, default=0)
    ps.add_argument("--concurrency", type=int, default=4)
    ps.add_argument("--queue-depth", type=int, default=16)
    ps.add_argument("--waiters", type=int, default=16)
    ps.add_argument("--max-context", type=int, default=8192)
    ps.add_argument("--seed", type=int, default=0)
    ps.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"])
    ps.add_argument("--engram-table", action="append", default=[],
                    help="flat Engram table file (loader.official.export_engram_table), once per Engram layer in layer "
                         "order; enables the Engram memory layers")
    ps.add_argument("--engram-random-rows", type=int, default=0,
                    help="random-init models: enable the Engram layers over random tables of this many rows")
    ps.add_argument("--speculative", action="store_true",
                    help="decode a lone greedy request with dSpark draft + verify rounds (random-init drafter unless the "
                         "checkpoint provides one)")
    args = ap.parse_args(argv)
    return {"build": cmd_build, "info": cmd_info, "serve": cmd_serve}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
