"""Small stand-alone cases of the non-GEMM hot kernels, for device timing and for profiler captures.

    python -m ds41rt_b200.utils.kernel_case                 # all cases, one JSON line
    python -m ds41rt_b200.utils.kernel_case --only attend_wide --reps 3

Cases (model-sized rows, working sets of a few hundred MB at most):
  attend_wide    sparse attention of a long pass: 256 rows x 64 heads x D 512, window 128 + 512 selected keys (bf16 rows)
  attend_decode  the same attention for 5 rows (key tiles split over CTAs); --attn-impl picks the kernel
  index_gemm     lightning-indexer scores on tensor cores: 1024 rows x 32 heads x 128 dims against 16384 keys
  topk           exact top-512 of 16384 scores for 1024 rows
  candidates     candidate-block selection: top 2048 blocks of 8 from 131072 scores for 64 rows
  sampler        GPU sampler: 8 rows x 129280 logits, temperature / top-k / top-p
Every case is timed with CUDA events after warm-up; algorithmic bytes or FLOPs per launch are stated beside the time.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from ..config import RopeConfig, rope_inv_freq
from ..ops import gemm as G
from ..ops import lib


def _time(fn, reps: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def attend_case(rows: int, heads: int = 64, D: int = 512, window: int = 128, topk: int = 512, ctx: int = 16384,
                impl: str = "tc"):
    k, dev = lib.kernels(), torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    ring, page_rows = window + max(16, rows), 64
    n_comp = ctx // 4
    max_pages = (n_comp + page_rows - 1) // page_rows
    win = torch.randn(1, ring, D, device=dev, generator=g).bfloat16()
    pool = torch.randn(max_pages * page_rows, D, device=dev, generator=g).bfloat16()
    page_table = torch.arange(max_pages, dtype=torch.int32, device=dev).view(1, max_pages).contiguous()
    pos = torch.arange(ctx - rows, ctx, dtype=torch.int32, device=dev)
    slot = torch.zeros(rows, dtype=torch.int32, device=dev)
    sel = torch.stack([torch.sort(torch.randperm(n_comp - 8, device=dev, generator=g)[:topk]).values
                       for _ in range(rows)]).int().contiguous()
    n_sel = torch.full((rows,), topk, dtype=torch.int32, device=dev)
    q = torch.randn(rows, heads * D, device=dev, generator=g).bfloat16()
    sink = torch.zeros(heads, device=dev)
    inv = torch.tensor(rope_inv_freq(RopeConfig(), 64), device=dev)
    from ..ops import attention as A
    if impl == "legacy":
        n_splits = max(1, min(16, -(-3 * 148 // (rows * ((heads + 15) // 16)))))
    else:
        n_splits = max(1, min((window + 16 + topk + 63) // 64, -(-2 * 148 // rows)))
    part_o = torch.zeros(rows, n_splits, heads, D, device=dev)
    part_ml = torch.zeros(rows, n_splits, heads, 2, device=dev)
    out = torch.zeros(rows, heads * D, device=dev, dtype=torch.bfloat16)
    status = lib.new_status(dev)

    def run():
        lib.check(A.attend(q=q, ldq=heads * D, q_off=0, rows=rows, heads=heads, D=D, window=window, ring=ring,
                           row_pos=pos, row_slot=slot, win=win, comp_pool=pool, sel=sel, n_sel=n_sel, k=topk,
                           page_table=page_table, max_pages=max_pages, page_rows=page_rows, inv_freq=inv, rope_dim=64,
                           scale=D ** -0.5, n_splits=n_splits, part_o=part_o, part_ml=part_ml, sink=sink, out=out,
                           ldo=heads * D, status=status, impl=impl), "attend")
    keys = window + topk
    flops = 2.0 * 2.0 * rows * heads * keys * D
    gathered = 2.0 * rows * keys * D          # each row's keys read once if all its heads share them
    return run, {"flops": flops, "bytes_min": gathered, "rows": rows, "keys_per_row": keys, "splits": n_splits,
                 "status": status}


def index_gemm_case(rows: int = 1024, n_keys: int = 16384, heads: int = 32, dim: int = 128):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    qr = torch.randn(rows * heads, dim, device=dev, generator=g).bfloat16()
    kc = torch.randn(n_keys, dim, device=dev, generator=g).bfloat16()
    w = torch.rand(rows, heads, device=dev, generator=g)
    vis = torch.full((rows,), n_keys, dtype=torch.int32, device=dev)
    scores = torch.zeros(rows, n_keys, device=dev)
    st = lib.new_status(dev)

    def run():
        G.gemm_raw(qr, kc, scores, rows * heads, n_keys, dim, lda=dim, ldb=dim, ldo=n_keys, out_mode=8, bn=256,
                   row_w=w, row_w_ld=heads, col_limit=vis, status=st)
    return run, {"flops": 2.0 * rows * heads * n_keys * dim, "bytes_min": 4.0 * rows * n_keys + 2.0 * n_keys * dim,
                 "scores": scores, "status": st}


def topk_case(scores: torch.Tensor, k_sel: int = 512):
    k, dev = lib.kernels(), scores.device
    rows, n = scores.shape
    pos = torch.full((rows,), n - 1, dtype=torch.int32, device=dev)
    slot = torch.zeros(rows, dtype=torch.int32, device=dev)
    sel = torch.zeros(rows, k_sel, dtype=torch.int32, device=dev)
    n_sel = torch.zeros(rows, dtype=torch.int32, device=dev)

    def run():
        lib.check(k.ds41_topk_select(lib.ptr(scores), n, lib.ptr(pos), lib.ptr(slot), 1, k_sel, lib.ptr(sel),
                                     lib.ptr(n_sel), rows, lib.stream()), "topk")
    return run, {"bytes_min": 4.0 * rows * n, "passes_over_scores": 6}


def candidates_case(rows: int = 64, n: int = 131072, block: int = 8, k_blocks: int = 2048):
    k, dev = lib.kernels(), torch.device("cuda")
    scores = torch.randn(rows, n, device=dev, generator=torch.Generator(device=dev).manual_seed(2))
    pos = torch.full((rows,), n - 1, dtype=torch.int32, device=dev)
    slot = torch.zeros(rows, dtype=torch.int32, device=dev)
    words = (n // block + 31) // 32
    blocks = torch.zeros(rows, k_blocks, dtype=torch.int32, device=dev)
    n_blocks = torch.zeros(rows, dtype=torch.int32, device=dev)
    mask = torch.zeros(rows, words, dtype=torch.int32, device=dev)

    def run():
        lib.check(k.ds41_candidate_select(lib.ptr(scores), n, lib.ptr(pos), lib.ptr(slot), 1, block, k_blocks,
                                          lib.ptr(blocks), lib.ptr(n_blocks), lib.ptr(mask), words, rows, lib.stream()),
                  "candidate_select")
    return run, {"bytes_min": 4.0 * rows * n, "passes_over_scores": 6}


def sampler_case(rows: int = 8, vocab: int = 129280):
    from ..ops.sampling import RowParams, pack_params, sample_rows
    dev = torch.device("cuda")
    logits = torch.randn(rows, vocab, device=dev, generator=torch.Generator(device=dev).manual_seed(3)) * 3
    params = pack_params([RowParams(temperature=0.8, top_k=50, top_p=0.9, seed=i) for i in range(rows)], dev)

    def run():
        sample_rows(logits, params)
    return run, {"bytes_min": 4.0 * rows * vocab}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--attn-impl", default="tc", choices=["tc", "legacy"],
                    help="attention cases: tcgen05 kernel (default) or the warp-MMA kernels")
    ap.add_argument("--attn-rows", type=int, default=256, help="rows of the attend_wide case")
    args = ap.parse_args(argv)
    want = lambda name: not args.only or name in args.only.split(",")
    out = {}
    idx = None
    if want("attend_wide"):
        run, info = attend_case(args.attn_rows, impl=args.attn_impl)
        ms = _time(run, args.reps)
        lib.raise_on_status(info.pop("status"), "attend_wide")
        out["attend_wide"] = {"ms": ms, "tflops": info["flops"] / ms / 1e9, "impl": args.attn_impl,
                              "gb_s_keys": info["bytes_min"] / ms / 1e6, **{k: v for k, v in info.items() if k != "flops"}}
    if want("attend_decode"):
        run, info = attend_case(5, impl=args.attn_impl)
        ms = _time(run, args.reps)
        lib.raise_on_status(info.pop("status"), "attend_decode")
        out["attend_decode"] = {"ms": ms, "gb_s_keys": info["bytes_min"] / ms / 1e6, "splits": info["splits"],
                                "impl": args.attn_impl}
    if want("index_gemm") or want("topk"):
        run, idx = index_gemm_case()
        ms = _time(run, args.reps)
        lib.raise_on_status(idx["status"], "index gemm")
        if want("index_gemm"):
            out["index_gemm"] = {"ms": ms, "tflops": idx["flops"] / ms / 1e9, "gb_s_out": idx["bytes_min"] / ms / 1e6}
    if want("topk"):
        run, info = topk_case(idx["scores"])
        ms = _time(run, args.reps)
        out["topk"] = {"ms": ms, "gb_s_one_pass": info["bytes_min"] / ms / 1e6}
    if want("candidates"):
        run, info = candidates_case()
        ms = _time(run, args.reps)
        out["candidates"] = {"ms": ms, "gb_s_one_pass": info["bytes_min"] / ms / 1e6}
    if want("sampler"):
        run, info = sampler_case()
        ms = _time(run, args.reps)
        out["sampler"] = {"ms": ms, "gb_s_one_pass": info["bytes_min"] / ms / 1e6}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
