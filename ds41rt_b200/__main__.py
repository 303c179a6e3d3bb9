"""Command line: `python -m ds41rt_b200 <command>`.

  build                      compile the kernel and host-runtime libraries in-tree
  serve  [--model ...]       OpenAI-compatible HTTP server over the native engine; under torch.distributed.run rank 0
                             serves and the other ranks mirror its engine calls (tensor + expert parallel)
  info                       print the model configuration and the per-rank memory plan
  doctor                     check the machine: toolchain, built libraries, GPUs, peer access, settings tiers
  inspect-model              tensor catalog of a configuration or a checkpoint directory (counts, bytes, placement)
  tokenize                   text -> token ids with the server's tokenizer
  load-tensors               read (and validate) tensors of a checkpoint, with timing
  plan-memory                KV page pool that fits a device next to the weights
  make-loadplan              which tensors (row / column ranges, bytes, experts) each rank reads from a checkpoint
  transport-capabilities     what the GPUs of this machine offer each other: peer access, NVLink, multicast, libraries
  scheduler-smoke            host-only check of admission, lanes, streaming and cancellation over a scripted backend
  selftest                   build and run the native self-test of the host runtime library (C ABI, no Python between)
  bench-kernels / campaign / prefill-matrix / validate-bench / convert-checkpoint / convert-engram-table
                             the tools of ds41rt_b200.utils, loader.convert and runtime.ple_convert under one entry
  select-gpus                which GPUs of this node have room for an N-rank launch (reads nvidia-smi only)
  source-manifest            write / verify the sha256 manifest of the source tree; identity of tree and toolchain
  release-report             results report (tables, scaling, clocks, provenance) recomputed from raw bench records
  audit-checkpoint           header-level audit of a checkpoint directory (structure, index agreement, identity digests)
  api-smoke                  protocol battery against a running server (health, chat, streaming, stop, seed, JSON, tools)

`serve` reads its options in three tiers: a KEY=VALUE settings file (`--settings`, default ./ds41rt.config), the
environment (DS41RT_<KEY>) and the command line, later tiers overriding earlier ones (ds41rt_b200/settings.py).

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


def cmd_doctor(args) -> int:
    """Machine check-up (reference: `ds41rt doctor`, rust/crates/ds41rt-daemon/src/cli.rs:15-35, scripts/doctor.sh)."""
    import shutil
    import subprocess
    from . import build
    rep = {"python": sys.version.split()[0]}
    try:
        import torch
        rep["torch"] = torch.__version__
        rep["cuda_available"] = torch.cuda.is_available()
        rep["gpus"] = []
        if torch.cuda.is_available():
            n = torch.cuda.device_count()
            for i in range(n):
                p = torch.cuda.get_device_properties(i)
                free, total = torch.cuda.mem_get_info(i)
                rep["gpus"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                    "memory_gb": round(total / 2 ** 30, 1), "free_gb": round(free / 2 ** 30, 1)})
            rep["peer_access"] = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)]
                                  for i in range(n)]
            rep["sm_100"] = all(g["sm"] == "10.0" for g in rep["gpus"])
        rep["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None
    except Exception as e:                                   # pragma: no cover - depends on the machine
        rep["torch_error"] = str(e)
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
    rep["nvcc"] = None
    if nvcc:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
        rep["nvcc"] = out.strip().splitlines()[-1] if out else nvcc
    rep["libraries"] = {n: (build.LIBDIR / n).exists() for n in ("libds41_kernels.so", "libds41_core.so")}
    rep["libraries_match_sources"] = {n: st["current"] for n, st in build.library_status().items()}
    rep["stale_sources"] = sorted(s for st in build.library_status().values() for s in st.get("stale", []))
    try:
        from .runtime import core as K
        K.core()
        rep["core_loads"] = True
    except Exception as e:
        rep["core_loads"] = f"{type(e).__name__}: {e}"
    from . import settings as S
    try:
        rep["settings_file"] = {"path": args.settings or (S.DEFAULT_FILE if os.path.exists(S.DEFAULT_FILE) else None),
                                "values": S.load_settings_file(args.settings or None)}
    except Exception as e:
        rep["settings_file"] = f"{type(e).__name__}: {e}"
    rep["environment"] = {k: v for k, v in os.environ.items() if k.startswith(S.ENV_PREFIX) or k.startswith("DS41_")}
    ok = bool(rep.get("cuda_available")) and all(rep["libraries"].values()) and rep.get("core_loads") is True
    rep["ok"] = ok
    print(json.dumps(rep, indent=1))
    return 0 if ok or args.lenient else 1


def cmd_inspect_model(args) -> int:
    """Catalog summary (reference: `ds41rt inspect-model`, rust/crates/ds41rt-loader/src/v41_catalog.rs:478-637)."""
    from .loader.catalog import Catalog, expected_tensors, official_templates
    cfg = _config(args)
    specs = expected_tensors(cfg, variant=args.variant)
    by_dtype, by_class = {}, {}
    import math
    sizes = {"BF16": 2, "F32": 4, "F8_E4M3": 1, "F8_E8M0": 1, "I8": 1, "U8": 1}
    for name, sp in specs.items():
        dt, shape = sp[0], sp[1]
        nbytes = math.prod(shape) * sizes.get(dt, 1)
        by_dtype[dt] = by_dtype.get(dt, 0) + nbytes
        cls = ("experts" if ".experts." in name else "shared_expert" if "shared_experts" in name else "attention"
               if ".attn." in name else "engram" if "engram" in name else "vision" if name.startswith("vision") else
               "drafter" if name.startswith("mtp.") else "other")
        by_class[cls] = by_class.get(cls, 0) + nbytes
    rep = {"model": cfg.name, "variant": args.variant, "tensors": len(specs),
           "templates": len(official_templates(cfg, args.variant)),
           "bytes_by_dtype": by_dtype, "gb_by_class": {k: round(v / 2 ** 30, 3) for k, v in by_class.items()},
           "total_gb": round(sum(by_dtype.values()) / 2 ** 30, 2)}
    if args.checkpoint:
        cat = Catalog(args.checkpoint, cfg, variant=args.variant)
        rep["checkpoint"] = {"directory": args.checkpoint, "shards": len(cat.files), "validated_tensors": len(cat.where)}
    if args.world > 1:
        # the Engram tables are read from host memory maps by rank 0 and never copied to a device as a whole
        tables = sum(math.prod(sp[1]) * sizes.get(sp[0], 1) for n, sp in specs.items() if ".engram.embed" in n)
        per_rank = by_class.get("experts", 0) / args.world + sum(v for k, v in by_class.items() if k != "experts") \
            - tables
        rep["per_rank_device_gb_expert_parallel"] = round(per_rank / 2 ** 30, 2)
        rep["host_engram_tables_gb"] = round(tables / 2 ** 30, 2)
    print(json.dumps(rep, indent=1))
    return 0


def cmd_tokenize(args) -> int:
    from .serving.tokenizer import ByteTokenizer, HFTokenizer
    cfg = _config(args)
    tk = HFTokenizer(args.tokenizer) if args.tokenizer else ByteTokenizer(vocab_size=cfg.vocab)
    text = args.text if args.text is not None else sys.stdin.read()
    ids = tk.encode(text)
    print(json.dumps({"tokens": len(ids), "ids": ids, "round_trip": tk.decode(ids) == text}))
    return 0


def cmd_load_tensors(args) -> int:
    """Read tensors of a checkpoint through the strict catalog (reference: `ds41rt load-tensors`)."""
    import fnmatch
    from .loader.catalog import Catalog
    cfg = _config(args)
    t0 = time.time()
    cat = Catalog(args.checkpoint, cfg, variant=args.variant)
    t_open = time.time() - t0
    names = [n for n in cat.where if fnmatch.fnmatch(n, args.pattern)][: args.limit or None]
    nbytes, t1 = 0, time.time()
    for n in names:
        t = cat.read(n)
        nbytes += t.numel() * t.element_size()
    dt = time.time() - t1
    print(json.dumps({"opened_s": round(t_open, 3), "tensors_read": len(names), "bytes": nbytes,
                      "read_s": round(dt, 3), "gb_per_s": round(nbytes / max(dt, 1e-9) / 1e9, 3)}))
    return 0


def cmd_plan_memory(args) -> int:
    from .runtime.memory import plan_pool
    cfg = _config(args)
    free = int(args.free_gb * 2 ** 30)
    plan = plan_pool(cfg, n_layers=cfg.n_layers, slots=args.concurrency, max_context=args.max_context,
                     free_bytes=free, kv_dtype=args.kv_dtype, retained=args.retained)
    print(json.dumps(plan.as_dict()))
    return 0


def _attach_engram(args, cfg, eng, dev):
    """Every rank: give the engine its Engram layers (checkpoint weights, or random ones for a random-init model).
    Returns the decoder layers that have one, in hash-family order."""
    if cfg.engram is None or not (args.engram_table or args.engram_random_rows):
        return []
    import torch
    from .models.engram import EngramLayer, init_engram_weights
    layers = [l for l in cfg.engram.layers if l < eng.n_layers]
    fmt = args.engram_format
    for i, l in enumerate(layers):
        scale = _engram_table_meta(args, i)["global_scale"]
        if args.checkpoint:
            from .loader.official import load_engram_layer
            mod = load_engram_layer(args.checkpoint, cfg, l, dev, table_format=fmt, table_scale=scale)
        else:
            wkv, q_w, k_w = init_engram_weights(cfg.hidden, seed=args.seed + 31 * i, std=0.002)
            bf = lambda t: t.to(device=dev, dtype=torch.bfloat16)
            mod = EngramLayer(bf(wkv), bf(q_w), bf(k_w), cfg.hidden, table_format=fmt, table_scale=scale)
        eng.attach_engram(l, mod)
    return layers


_random_tables: dict = {}


def _random_engram_table(args, i: int) -> dict:
    """A small random table for a random-init model, written once per process (and converted when the format asks for
    it): {"path", "row_bytes", "global_scale"}.  Every rank derives the same scale from the same seed."""
    key = (args.seed, i, args.engram_random_rows, args.engram_format)
    if key not in _random_tables:
        import tempfile
        from .models.engram import random_table_rows
        path = os.path.join(tempfile.mkdtemp(prefix="ds41-engram-"), f"table{i}.bin")
        random_table_rows(args.engram_random_rows, seed=args.seed + i).numpy().tofile(path)
        meta = {"path": path, "row_bytes": 264, "global_scale": 1.0}
        if args.engram_format == "nvfp4":
            from .runtime.ple_convert import convert_table
            done = convert_table(path, path + ".nvfp4", args.engram_random_rows)
            meta = {"path": path + ".nvfp4", "row_bytes": done["row_bytes"], "global_scale": done["global_scale"]}
        _random_tables[key] = meta
    return _random_tables[key]


def cmd_make_loadplan(args) -> int:
    """Per-rank load plan (reference: `ds41rt make-loadplan`, rust/crates/ds41rt-loader/src/v41_catalog.rs:215-273)."""
    import math
    from .loader.catalog import Catalog, expected_tensors
    cfg = _config(args)
    sizes = {"BF16": 2, "F32": 4, "F8_E4M3": 1, "F8_E8M0": 1, "I8": 1, "U8": 1}
    if args.checkpoint:
        cat = Catalog(args.checkpoint, cfg, variant=args.variant)
    else:                                                    # plan from the configuration alone
        cat = object.__new__(Catalog)
        cat.cfg, cat.expected = cfg, expected_tensors(cfg, args.variant)
    ranks = [args.rank] if args.rank >= 0 else list(range(args.world))
    out = {"model": cfg.name, "variant": args.variant, "world": args.world, "ranks": []}
    for r in ranks:
        plan = cat.shard_plan(r, args.world)
        total, tables, sliced, experts = 0, 0, 0, set()
        for name, (rows, cols) in plan.items():
            dt, shape = cat.expected[name][0], list(cat.expected[name][1])
            if rows is not None and shape:
                shape[0] = rows[1] - rows[0]
            if cols is not None and len(shape) > 1:
                shape[1] = cols[1] - cols[0]
            if ".engram.embed" in name:                  # memory-mapped on the host of rank 0, gathered row by row
                tables += math.prod(shape) * sizes.get(dt, 1)
                continue
            total += math.prod(shape) * sizes.get(dt, 1)
            sliced += rows is not None or cols is not None
            if ".ffn.experts." in name and not name.startswith("mtp."):
                parts = name.split(".")
                experts.add(int(parts[parts.index("experts") + 1]))
        entry = {"rank": r, "tensors": len(plan), "sliced_tensors": sliced, "device_gb": round(total / 2 ** 30, 3),
                 "host_engram_tables_gb": round(tables / 2 ** 30, 3) if r == 0 else 0.0,
                 "experts": [min(experts), max(experts)] if experts else None}
        if args.list:
            entry["plan"] = {n: {"rows": rc[0], "cols": rc[1]} for n, rc in plan.items()}
        out["ranks"].append(entry)
    print(json.dumps(out, indent=None if args.list else 1))
    return 0


def cmd_transport_capabilities(args) -> int:
    """What the GPUs offer each other (reference: `ds41rt transport-capabilities`, which reports its TCP / RDMA paths;
    here the transport is NVLink peer memory, so the report is about that).  Read-only."""
    rep = {"transport": "peer memory over NVLink / NVSwitch (loads, stores and multimem from inside kernels); NCCL for "
                        "bootstrap and baselines"}
    try:
        import torch
        rep["cuda_available"] = torch.cuda.is_available()
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        rep["gpus"] = n
        rep["peer_access"] = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)]
                              for i in range(n)]
        rep["all_peers"] = all(all(row) for row in rep["peer_access"]) if n else False
        rep["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if n else None
        rep["multimem_capable"] = bool(n) and all(torch.cuda.get_device_capability(i)[0] >= 9 for i in range(n))
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
            rep["symmetric_memory"] = True
        except Exception as e:
            rep["symmetric_memory"] = f"{type(e).__name__}: {e}"
    except Exception as e:                                   # pragma: no cover - depends on the machine
        rep["torch_error"] = str(e)
    try:
        import pynvml
        pynvml.nvmlInit()
        links = []
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            up = 0
            for l in range(18):
                try:
                    up += int(pynvml.nvmlDeviceGetNvLinkState(h, l) == 1)
                except pynvml.NVMLError:
                    break
            links.append(up)
        rep["nvlink_links_up"] = links
        pynvml.nvmlShutdown()
    except Exception as e:
        rep["nvlink_links_up"] = f"unavailable ({type(e).__name__})"
    rep["environment"] = {k: os.environ[k] for k in ("NCCL_NVLS_ENABLE", "NCCL_P2P_DISABLE", "CUDA_VISIBLE_DEVICES")
                          if k in os.environ}
    print(json.dumps(rep, indent=1))
    return 0


def cmd_scheduler_smoke(args) -> int:
    """Host-only smoke of the serving path over a scripted backend: bounded admission, lane balance, a streamed and a
    plain completion through the real HTTP server, and a cancelled stream (reference: `ds41rt scheduler-smoke`)."""
    import http.client
    from .runtime import core as K
    from .serving.engine import FakeBackend
    from .serving.http import ApiServer
    from .serving.tokenizer import ByteTokenizer
    rep = {}
    adm = K.Admission(2, 1)
    got = [adm.reserve() for _ in range(4)]              # 0 queued, 1 waiting, -1 refused
    rep["admission"] = {"entered": sum(1 for g in got if g >= 0), "refused": sum(1 for g in got if g < 0)}
    lanes = K.Lanes(2)
    placed = [lanes.add(i, 100 + i, 10) for i in range(4)]
    rep["lanes"] = {"placed": placed, "loads": [lanes.load(0), lanes.load(1)]}
    tk = ByteTokenizer()
    script = tk.encode("scheduler smoke ok")
    srv = ApiServer(FakeBackend(script, tk, delay=0.001), tk, queue_depth=4, waiters=4).start()
    try:
        body = {"model": "deepseek-ai/DeepSeek-V4.1-Flash", "messages": [{"role": "user", "content": "hi"}],
                "max_tokens": 32, "thinking": {"type": "disabled"}}
        hdr = {"Content-Type": "application/json", "Connection": "close"}
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=30)
        c.request("POST", "/v1/chat/completions", body=json.dumps(body).encode(), headers=hdr)
        r = c.getresponse()
        doc = json.loads(r.read())
        rep["plain"] = {"status": r.status, "text": doc["choices"][0]["message"]["content"] if r.status == 200 else doc}
        c.close()
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=30)
        c.request("POST", "/v1/chat/completions", body=json.dumps(dict(body, stream=True)).encode(), headers=hdr)
        r = c.getresponse()
        lines = [l for l in r.read().split(b"\n") if l.startswith(b"data: ")]
        rep["stream"] = {"status": r.status, "events": len(lines), "done": lines[-1].strip() == b"data: [DONE]"}
        c.close()
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=30)
        c.request("GET", "/health", headers={"Connection": "close"})
        r = c.getresponse()
        r.read()
        rep["health"] = r.status
        c.close()
    finally:
        srv.stop()
    ok = rep["admission"] == {"entered": 3, "refused": 1} and rep["plain"]["status"] == 200 \
        and rep["plain"]["text"] == "scheduler smoke ok" and rep["stream"]["done"] and rep["health"] == 200
    rep["ok"] = bool(ok)
    print(json.dumps(rep, indent=1))
    return 0 if ok else 1


def cmd_selftest(args) -> int:
    """Native self-test of libds41_core.so (csrc/tests/core_selftest.cc); exit status = failed checks."""
    import subprocess
    from . import build
    exe = build.build_selftest()
    return subprocess.run([str(exe)]).returncode


def _forward(module: str):
    def run(args) -> int:
        import importlib
        rest = args.rest[1:] if args.rest[:1] == ["--"] else args.rest
        return int(importlib.import_module(module, __package__).main(rest) or 0)
    return run


FORWARDED = {"bench-kernels": ".utils.kernel_case", "campaign": ".utils.http_campaign",
             "prefill-matrix": ".utils.prefill_matrix", "validate-bench": ".utils.validate_bench",
             "convert-checkpoint": ".loader.convert", "convert-engram-table": ".runtime.ple_convert",
             "engram-io-bench": ".runtime.engram_io", "select-gpus": ".utils.select_gpus",
             "source-manifest": ".utils.source_manifest", "release-report": ".utils.release_report",
             "api-smoke": ".utils.api_smoke", "audit-checkpoint": ".loader.audit"}


def _engram_table_meta(args, i: int) -> dict:
    """Record size and table scale of the i-th table: from the `.json` that runtime.ple_convert wrote beside a converted
    table, the fixed 264-byte FP8 record otherwise."""
    if not args.engram_table:
        return _random_engram_table(args, i)
    if args.engram_format != "nvfp4":
        return {"path": args.engram_table[i], "row_bytes": 264, "global_scale": 1.0}
    with open(args.engram_table[i] + ".json") as f:
        meta = json.load(f)
    if meta.get("format") != "nvfp4" or not meta.get("complete"):
        raise SystemExit(f"{args.engram_table[i]}: not a finished NVFP4 conversion")
    return {"path": args.engram_table[i], "row_bytes": meta["row_bytes"], "global_scale": meta["global_scale"]}


def _engram_pipeline(args, cfg, eng, layers, tokenizer):
    """Rank 0: the tables and the gather threads behind the engine's Engram layers."""
    if not layers:
        return None
    from .runtime.engram import EngramPipeline, compressed_token_ids
    from .runtime.engram_io import EngramTable
    tables = []
    for i, l in enumerate(layers):
        meta = _engram_table_meta(args, i)
        # a checkpoint's table has the configured row count; a random table is small and row ids are folded into it
        n_rows = (cfg.engram.num_embeddings[cfg.engram.layers.index(l)] if args.engram_table
                  else args.engram_random_rows)
        tables.append(EngramTable(meta["path"], n_rows, meta["row_bytes"]))
    return EngramPipeline(layers, tables, token_map=compressed_token_ids(tokenizer.token_bytes()),
                          pad_id=cfg.engram.pad_token_id, max_rows=eng.max_rows, fold=not args.engram_table)


def _vision_tower(args, cfg, dev):
    """(VisionTower, VisionConfig) for `serve --vision`: the checkpoint's `vision.*` / `aligner.*` tensors, or random
    weights of a small tower for a random-init model."""
    from .config import VisionConfig
    from .models.vision import VisionTower, init_vision_weights
    if args.checkpoint:
        from .loader.catalog import Catalog
        v = cfg.vision or VisionConfig()
        cat = Catalog(args.checkpoint, cfg, with_vision=True, with_engram=cfg.engram is not None)
        weights = {n: cat.read(n).float() for n in cat.where if n.startswith(("vision.", "aligner."))}
        return VisionTower(v, weights, cfg.hidden, v.layers, dev), v
    v = VisionConfig(layers=2, hidden=256, heads=4, intermediate=384, min_pixels=42 * 42 * 4, max_image_tokens=64)
    weights = init_vision_weights(v, cfg.hidden, v.layers, seed=args.seed + 5, std=0.05)
    return VisionTower(v, weights, cfg.hidden, v.layers, dev, max_patches=(v.max_image_tokens * v.downsample ** 2)), v


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
    image_marks = ["<image>", "<image_start>", "<image_end>", "<image_newline>"]
    tk = HFTokenizer(args.tokenizer) if args.tokenizer else \
        ByteTokenizer(vocab_size=cfg.vocab, extra_specials=image_marks if args.vision else ())
    t0 = time.time()
    if args.checkpoint:
        from .loader.official import load_engine_weights
        weights = load_engine_weights(args.checkpoint, cfg, rank, world, dev, expert_dtype=args.expert_dtype)
    else:
        weights = EngineWeights.random(cfg, rank, world, dev, seed=args.seed, expert_dtype=args.expert_dtype)
    # KV pool: what the request slots want at full context, cut to what is free beside the weights
    from .runtime.memory import plan_pool
    torch.cuda.synchronize()
    free_now = torch.cuda.mem_get_info(dev)[0]
    plan = plan_pool(cfg, n_layers=cfg.n_layers, slots=args.concurrency, max_context=args.max_context,
                     free_bytes=free_now, kv_dtype=args.kv_dtype, retained=args.prompt_snapshots + args.turn_snapshots,
                     ring_rows=cfg.window + max(16, args.prefill_chunk), reserve_bytes=args.reserve_gb << 30)
    n_pages = int(fabric.all_reduce_max(-plan.pages) * -1) if world > 1 else plan.pages     # the smallest rank decides
    if n_pages < (args.max_context + 63) // 64 + 1:
        print(f"rank {rank}: only {n_pages} KV pages fit; lower --max-context or --concurrency", file=sys.stderr)
        return 2
    eng = DS41Engine(cfg, weights, fabric, max_rows=max(8, args.concurrency, args.prefill_chunk), slots=args.concurrency,
                     max_ctx=args.max_context, kv_dtype=args.kv_dtype, n_pages=n_pages)
    engram_layers = _attach_engram(args, cfg, eng, dev)
    hb = None
    if world > 1:
        # liveness over a TCP store next to the rendezvous port: heartbeats from every rank, a guard on the leader
        import torch.distributed as dist
        from .parallel.health import Heartbeat
        port = int(os.environ.get("MASTER_PORT", "29500")) + 7
        store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), port, world, is_master=(rank == 0),
                              wait_for_workers=False)
        hb = Heartbeat(store, rank, world, interval=0.5, max_age=args.peer_timeout).start()
        hb.wait_joined(60.0)
    if rank != 0:
        # every other rank mirrors the leader's engine calls until it is told to stop
        follower_loop(eng, ctl, on_error=lambda e: print(f"rank {rank}: {e}", file=sys.stderr, flush=True), heartbeat=hb)
        return 0
    lead = LeaderEngine(eng, ctl, heartbeat=hb)
    tower = vision_cfg = None
    if args.vision:
        # image parts of chat messages: the tower runs on the serving rank and its rows replace placeholder embeddings
        if world > 1:
            print("--vision serves from one rank only in this build; ignoring it", file=sys.stderr)
        else:
            tower, vision_cfg = _vision_tower(args, cfg, dev)
    drafter = None
    if args.speculative:
        if world > 1:
            print("--speculative serves from one rank only in this build; ignoring it", file=sys.stderr)
        else:
            from .models.dspark import DSparkDrafter
            drafter = DSparkDrafter(cfg, eng, weights=None, seed=args.seed, expert_dtype=args.expert_dtype)
    backend = NativeBackend(lead if world > 1 else eng, eos=tk.eos, concurrency=args.concurrency,
                            queue_depth=args.queue_depth, drafter=drafter, prefill_chunk=args.prefill_chunk,
                            prompt_snapshots=args.prompt_snapshots, turn_snapshots=args.turn_snapshots,
                            host_cache_bytes=int(args.host_cache_gb * (1 << 30)) if world == 1 else 0,
                            engram=_engram_pipeline(args, cfg, eng, engram_layers, tk), vision=tower)
    srv = ApiServer(backend, tk, host=args.host, port=args.port, queue_depth=args.queue_depth, waiters=args.waiters,
                    max_context=args.max_context, vision_cfg=vision_cfg).start()
    print(json.dumps({"listening": f"http://{args.host}:{srv.port}", "model": cfg.name, "ranks": world,
                      "setup_s": round(time.time() - t0, 1), "kv_pool": plan.as_dict() | {"pages": n_pages},
                      "settings": {k: v for k, v in getattr(args, "_origin", {}).items() if v != "default"}}), flush=True)
    # SIGTERM (./stop.sh, a container runtime) ends the server the way Ctrl-C does: the listener closes, the worker
    # drains, and the mirroring ranks are told to stop instead of waiting for a leader that vanished
    import signal

    def _terminate(signum, frame):
        raise KeyboardInterrupt

    signal.signal(signal.SIGTERM, _terminate)
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
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in FORWARDED:                         # a tool parses its own options, leading flags included
        import importlib
        rest = argv[2:] if argv[1:2] == ["--"] else argv[1:]
        return int(importlib.import_module(FORWARDED[argv[0]], __package__).main(rest) or 0)
    ap = argparse.ArgumentParser(prog="ds41rt_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def model_args(p):
        p.add_argument("--model", default="tiny", choices=["tiny", "small", "flash"])
        p.add_argument("--layers", type=int, default=0, help="flash: number of layers to instantiate")
        p.add_argument("--config", default="", help="official config.json (overrides --model)")

    sub.add_parser("build")
    pi = sub.add_parser("info")
    model_args(pi)
    pd = sub.add_parser("doctor")
    pd.add_argument("--settings", default="", help="settings file to check (default ./ds41rt.config when present)")
    pd.add_argument("--lenient", action="store_true", help="exit 0 even when a check fails (report only)")
    pm = sub.add_parser("inspect-model")
    model_args(pm)
    pm.add_argument("--variant", default="mxfp4", choices=["mxfp4", "nvfp4"])
    pm.add_argument("--checkpoint", default="", help="validate this checkpoint directory against the catalog")
    pm.add_argument("--world", type=int, default=1, help="ranks: also print the per-rank share under expert parallelism")
    pt = sub.add_parser("tokenize")
    model_args(pt)
    pt.add_argument("--tokenizer", default="")
    pt.add_argument("--text", default=None, help="text to encode (default: standard input)")
    pl = sub.add_parser("load-tensors")
    model_args(pl)
    pl.add_argument("--checkpoint", required=True)
    pl.add_argument("--variant", default="mxfp4", choices=["mxfp4", "nvfp4"])
    pl.add_argument("--pattern", default="*", help="shell pattern over tensor names")
    pl.add_argument("--limit", type=int, default=0)
    pp = sub.add_parser("plan-memory")
    model_args(pp)
    pp.add_argument("--free-gb", type=float, required=True, help="device memory left after the weights")
    pp.add_argument("--concurrency", type=int, default=4)
    pp.add_argument("--max-context", type=int, default=8192)
    pp.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"])
    pp.add_argument("--retained", type=int, default=40)
    pk = sub.add_parser("make-loadplan")
    model_args(pk)
    pk.add_argument("--checkpoint", default="", help="validate against this checkpoint (default: plan from the configuration)")
    pk.add_argument("--variant", default="mxfp4", choices=["mxfp4", "nvfp4"])
    pk.add_argument("--world", type=int, default=8)
    pk.add_argument("--rank", type=int, default=-1, help="only this rank (default: all)")
    pk.add_argument("--list", action="store_true", help="include every tensor with its row / column range")
    sub.add_parser("transport-capabilities")
    sub.add_parser("scheduler-smoke")
    sub.add_parser("selftest")
    for name in FORWARDED:
        pf = sub.add_parser(name, add_help=False)
        pf.add_argument("rest", nargs=argparse.REMAINDER)
    ps = sub.add_parser("serve")
    model_args(ps)
    ps.add_argument("--settings", default="", help="KEY=VALUE settings file (default ./ds41rt.config when present)")
    ps.add_argument("--prefill-chunk", type=int, default=2048, help="rows per prompt pass (80-4096)")
    ps.add_argument("--prompt-snapshots", type=int, default=20, help="prompt-bank capacity (LRU)")
    ps.add_argument("--turn-snapshots", type=int, default=20, help="turn-bank capacity (LRU)")
    ps.add_argument("--host-cache-gb", type=float, default=0.0,
                    help="pinned host memory for snapshots that leave the device banks (0 = off; one-rank serving)")
    ps.add_argument("--reserve-gb", type=int, default=0, help="device memory to leave untouched by the KV pool")
    ps.add_argument("--peer-timeout", type=float, default=10.0, help="seconds without a heartbeat before a rank counts as gone")
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
    ps.add_argument("--engram-format", default="fp8", choices=["fp8", "nvfp4"],
                    help="record format of the --engram-table files: fp8 (264-byte records as exported) or nvfp4 "
                         "(144-byte records written by `python -m ds41rt_b200.runtime.ple_convert`, with the table "
                         "scale read from FILE.json)")
    ps.add_argument("--engram-random-rows", type=int, default=0,
                    help="random-init models: enable the Engram layers over random tables of this many rows")
    ps.add_argument("--vision", action="store_true",
                    help="accept image parts in chat messages: vision tower from the checkpoint (or a small random one "
                         "for a random-init model); one-rank serving")
    ps.add_argument("--speculative", action="store_true",
                    help="decode with dSpark draft + verify rounds: a lone request, or up to four active requests sharing "
                         "a round (random-init drafter unless the checkpoint provides one)")
    argv = list(sys.argv[1:] if argv is None else argv)
    args = ap.parse_args(argv)
    if args.cmd == "serve":
        # settings tiers: file < environment < command line
        from . import settings as S
        file_values = S.load_settings_file(args.settings or None)
        args = S.apply_tiers(ps, argv[argv.index("serve") + 1:], file_values)
        args.cmd = "serve"
        if not 80 <= args.prefill_chunk <= 4096:
            ap.error("--prefill-chunk must be within 80..4096")
        if not 1 <= args.concurrency <= 64:
            ap.error("--concurrency must be within 1..64")
    table = {"build": cmd_build, "info": cmd_info, "serve": cmd_serve, "doctor": cmd_doctor,
             "inspect-model": cmd_inspect_model, "tokenize": cmd_tokenize, "load-tensors": cmd_load_tensors,
             "plan-memory": cmd_plan_memory, "make-loadplan": cmd_make_loadplan,
             "transport-capabilities": cmd_transport_capabilities, "scheduler-smoke": cmd_scheduler_smoke,
             "selftest": cmd_selftest}
    table.update({name: _forward(mod) for name, mod in FORWARDED.items()})
    return table[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
