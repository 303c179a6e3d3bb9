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
  router         gate projection (384 experts x 5120) + sqrt-softplus top-6 selection, 5 rows and 2048 rows
  hc             hyper-connection boundary (expand, mixes, collapse, RMSNorm) of 4 x 5120 streams, 5 rows and 2048 rows
`--impl reference` runs the reference's own kernels for the cases it has a counterpart of (attention, top-k, router,
hc, indexer scores) through `utils/reference_arm.py`; `--kv fp8fp4` gives this package's attention the same cache row
formats as that arm (FP8 window rows, FP4 compressed rows).
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


def _fp8_rows(x: torch.Tensor, row_bytes: int) -> torch.Tensor:
    """bf16 rows -> cache rows of E4M3 values followed by one E8M0 scale per 32 values."""
    from ..ops import quant_ref as Q
    D = x.shape[-1]
    q, e = Q.quant_mxfp8(x.float(), 32)
    rows = torch.zeros(*x.shape[:-1], row_bytes, dtype=torch.uint8, device=x.device)
    rows[..., :D] = q.view(torch.uint8)
    rows[..., D:D + D // 32] = e.to(torch.uint8)
    return rows.contiguous()


def _fp4_rows(x: torch.Tensor, row_bytes: int) -> torch.Tensor:
    """bf16 rows -> cache rows of E2M1 pairs followed by one E4M3 scale per 16 values."""
    from ..ops import quant_ref as Q
    D = x.shape[-1]
    packed, bs = Q.quant_kv_fp4_e4m3_16(x.float())
    rows = torch.zeros(*x.shape[:-1], row_bytes, dtype=torch.uint8, device=x.device)
    rows[..., :D // 2] = packed.view(torch.uint8).reshape(*x.shape[:-1], D // 2)
    rows[..., D // 2:D // 2 + D // 16] = bs.view(torch.uint8).reshape(*x.shape[:-1], D // 16)
    return rows.contiguous()


def attend_case(rows: int, heads: int = 64, D: int = 512, window: int = 128, topk: int = 512, ctx: int = 16384,
                impl: str = "tc", kv: str = "bf16"):
    k, dev = lib.kernels(), torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    ring, page_rows = window + max(16, rows), 64
    n_comp = ctx // 4
    max_pages = (n_comp + page_rows - 1) // page_rows
    win = torch.randn(1, ring, D, device=dev, generator=g).bfloat16()
    pool = torch.randn(max_pages * page_rows, D, device=dev, generator=g).bfloat16()
    row_bytes = comp_bytes = 0
    if kv == "fp8fp4":
        row_bytes, comp_bytes = (D + D // 32 + 15) // 16 * 16, (D // 2 + D // 16 + 15) // 16 * 16
        win, pool = _fp8_rows(win, row_bytes), _fp4_rows(pool, comp_bytes)
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
                           ldo=heads * D, kv_row_bytes=row_bytes, comp_row_bytes=comp_bytes, status=status, impl=impl),
                  "attend")
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


def router_case(rows: int, experts: int = 384, H: int = 5120):
    """Split-K gate projection on tensor cores, then one selection kernel (sums the planes, sqrt-softplus, top 6)."""
    k, dev = lib.kernels(), torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    hidden = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    weight = (torch.randn(experts, H, device=dev, generator=g) * H ** -0.5).bfloat16()
    bias = torch.randn(experts, device=dev, generator=g) * 0.01
    bn = G.pick_bn(rows)
    splits = G.pick_splits(experts, H, max_splits=16, n_tiles=(rows + bn - 1) // bn)
    planes = torch.zeros(splits, rows, experts, device=dev)
    ids = torch.zeros(rows, 6, dtype=torch.int32, device=dev)
    wts = torch.zeros(rows, 6, device=dev)
    st = lib.new_status(dev)

    def run():
        G.linear_planes(hidden, weight, planes, splits, status=st)
        lib.check(k.ds41_router_select(lib.ptr(planes), splits, rows, experts, experts, 0, 6, lib.ptr(bias),
                                       C.c_float(1.5), C.c_float(10.0), lib.ptr(ids), lib.ptr(wts), lib.ptr(None),
                                       lib.stream()), "router_select")
    return run, {"flops": 2.0 * rows * experts * H, "splits": splits, "status": st, "ids": ids, "weights": wts}


def hc_case(rows: int, H: int = 5120):
    """Expand with the sublayer's output plane, next mixes, collapse and RMSNorm: one fused launch up to 16 rows, two
    kernels for long passes."""
    k, dev = lib.kernels(), torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    streams = torch.randn(rows, 4, H, device=dev, generator=g).bfloat16()
    sub = torch.randn(1, rows, H, device=dev, generator=g)
    fn = torch.randn(24, 4 * H, device=dev, generator=g) * 0.02
    scale = torch.tensor([1.0, 0.7, 1.3], device=dev)
    base = torch.randn(24, device=dev, generator=g) * 0.5
    pre_in = torch.rand(rows, 4, device=dev, generator=g)
    post = torch.rand(rows, 4, device=dev, generator=g)
    comb = torch.rand(rows, 16, device=dev, generator=g)
    norm_w = torch.rand(H, device=dev, generator=g) + 0.5
    st = lib.new_status(dev)
    bases = (C.c_void_p * 1)(sub.data_ptr())
    out_streams = torch.zeros_like(streams)
    next_pre, post2 = torch.zeros(rows, 4, device=dev), torch.zeros(rows, 4, device=dev)
    comb2 = torch.zeros(rows, 16, device=dev)
    xn = torch.zeros(rows, H, device=dev, dtype=torch.bfloat16)
    if rows <= 16:
        partial = torch.zeros(H // 128, rows, 26, device=dev)
        xc = torch.zeros(rows, H, device=dev)
        tickets = torch.zeros(rows, dtype=torch.int32, device=dev)
        a = lib.HcStepArgs()
        a.streams_in, a.streams_out = lib.ptr(streams), lib.ptr(out_streams)
        a.part_bases = C.cast(bases, C.c_void_p)
        a.post, a.comb, a.pre_in = lib.ptr(post), lib.ptr(comb), lib.ptr(pre_in)
        a.fn, a.scale, a.base, a.norm_w = lib.ptr(fn), lib.ptr(scale), lib.ptr(base), lib.ptr(norm_w)
        a.partial, a.xc = lib.ptr(partial), lib.ptr(xc)
        a.next_pre, a.post_out, a.comb_out, a.xn = lib.ptr(next_pre), lib.ptr(post2), lib.ptr(comb2), lib.ptr(xn)
        a.tickets, a.status = lib.ptr(tickets), lib.ptr(st)
        a.split_stride, a.n_ranks, a.n_splits = rows * H, 1, 1
        a.rows, a.H, a.iters, a.hc_eps, a.norm_eps = rows, H, 20, 1e-6, 1e-20
        keep = (partial, xc, tickets)

        def run():
            lib.check(k.ds41_hc_step(C.byref(a), lib.stream()), "hc_step")
    else:
        partial = torch.zeros(H // 128, rows, 25, device=dev)
        keep = (partial,)

        def run():
            lib.check(k.ds41_hc_post_mix(lib.ptr(streams), lib.ptr(out_streams), bases, 1, 1, C.c_longlong(rows * H),
                                         lib.ptr(post), lib.ptr(comb), lib.ptr(fn), lib.ptr(partial), rows, H,
                                         lib.ptr(None), lib.ptr(None), lib.ptr(st), lib.ptr(None), lib.ptr(None), lib.ptr(None), lib.ptr(None), C.c_float(0.0), lib.stream()),
                      "hc_post_mix")
            lib.check(k.ds41_hc_finish(lib.ptr(partial), H // 128, lib.ptr(scale), lib.ptr(base), lib.ptr(pre_in),
                                       lib.ptr(out_streams), lib.ptr(norm_w), lib.ptr(next_pre), lib.ptr(post2),
                                       lib.ptr(comb2), lib.ptr(xn), lib.ptr(None), lib.ptr(None), lib.ptr(None), rows, H,
                                       20, C.c_float(1e-6), C.c_float(1e-20), lib.ptr(None), 0, C.c_longlong(0), 0,
                                       lib.stream()), "hc_finish")
    streams_bytes = 2.0 * rows * 4 * H
    return run, {"bytes_min": 2 * streams_bytes + 4.0 * rows * H + 2.0 * rows * H + 4.0 * 24 * 4 * H, "status": st,
                 "keep": (keep, streams, sub, fn, scale, base, pre_in, post, comb, norm_w, out_streams, next_pre, post2,
                          comb2, xn, bases)}


def reference_main(args) -> int:
    """One JSON line of the reference's own kernels at the shapes of the cases above."""
    from . import reference_arm as REF
    if REF.library() is None:
        print(json.dumps({"impl": "reference", "unavailable": REF.why()}))
        return 0
    want = lambda name: not args.only or name in args.only.split(",")
    out = {"impl": "reference"}
    if want("attend_wide"):
        run, info = REF.attention_case(args.attn_rows, check_rows=2)
        ms = _time(run, args.reps)
        out["attend_wide"] = {"ms": ms, "tflops": info["flops"] / ms / 1e9, "rows": info["rows"], "entry": info["entry"],
                              "keys_per_row": info["keys_per_row"], "max_rel_err_vs_fp32": info["max_rel_err_vs_fp32"]}
    if want("attend_decode"):
        run, info = REF.attention_case(5, check_rows=2)
        ms = _time(run, args.reps)
        out["attend_decode"] = {"ms": ms, "entry": info["entry"], "max_rel_err_vs_fp32": info["max_rel_err_vs_fp32"]}
    if want("index_gemm"):
        run, info = REF.index_case()
        ms = _time(run, max(1, args.reps // 4))
        out["index_gemm"] = {"ms": ms, "tflops": info["flops"] / ms / 1e9, "queries": info["queries"],
                             "candidates": info["candidates"], "ns_per_score": ms * 1e6 / (info["queries"] * info["candidates"])}
    if want("topk"):
        run, info = REF.topk_case()
        ms = _time(run, args.reps)
        out["topk"] = {"ms": ms, "gb_s_one_pass": info["bytes_min"] / ms / 1e6}
    if want("sampler"):
        # same logits, seeds and filters as this package's `sampler` case; both samplers implement the same host oracle,
        # so their tokens can be compared
        from ..runtime import core
        run, info = REF.sampler_case()
        ms = _time(run, args.reps)
        tok, st = info["tokens"].cpu().tolist(), info["status"].cpu().tolist()
        lg = info["logits"].cpu().numpy()
        agree = sum(int(st[r] == 0 and tok[r] == core.sample_token(lg[r], None, 0.8, 50, 0.9, 0.0,
                                                                    core.sample_uniform(r, 0))) for r in range(len(tok)))
        out["sampler"] = {"ms": ms, "gb_s_one_pass": info["bytes_min"] / ms / 1e6, "kernels": "K1 + K2, K3 + K4, K5",
                          "status_ok_rows": sum(int(x == 0) for x in st), "tokens_equal_to_host_oracle": f"{agree}/{len(tok)}"}
    for name, rows in (("router_decode", 5), ("router_wide", 2048)):
        if want(name) or want("router"):
            run, info = REF.router_case(rows)
            ms = _time(run, args.reps)
            out[name] = {"ms": ms, "rows": rows, "tflops": info["flops"] / ms / 1e9}
    for name, rows in (("hc_decode", 5), ("hc_wide", 2048)):
        if want(name) or want("hc"):
            run, info = REF.hc_case(rows)
            ms = _time(run, args.reps)
            out[name] = {"ms": ms, "rows": rows, "gb_s": info["bytes_min"] / ms / 1e6,
                         "kernels": "hc_post + hc_mixes + hc_pre (RMSNorm not included)"}
    print(json.dumps(out))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--attn-impl", default="tc", choices=["tc", "legacy"],
                    help="attention cases: tcgen05 kernel (default) or the warp-MMA kernels")
    ap.add_argument("--attn-rows", type=int, default=256, help="rows of the attend_wide case")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8fp4"],
                    help="attention cases: cache row formats (fp8fp4 = FP8 window rows + FP4 compressed rows)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_main(args)
    want = lambda name: not args.only or name in args.only.split(",")
    out = {}
    idx = None
    if want("attend_wide"):
        run, info = attend_case(args.attn_rows, impl=args.attn_impl, kv=args.kv)
        ms = _time(run, args.reps)
        lib.raise_on_status(info.pop("status"), "attend_wide")
        out["attend_wide"] = {"ms": ms, "tflops": info["flops"] / ms / 1e9, "impl": args.attn_impl,
                              "kv": args.kv, "gb_s_keys": info["bytes_min"] / ms / 1e6,
                              **{k: v for k, v in info.items() if k != "flops"}}
    if want("attend_decode"):
        run, info = attend_case(5, impl=args.attn_impl, kv=args.kv)
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
    for name, rows in (("router_decode", 5), ("router_wide", 2048)):
        if want(name) or want("router"):
            run, info = router_case(rows)
            ms = _time(run, args.reps)
            lib.raise_on_status(info["status"], name)
            out[name] = {"ms": ms, "rows": rows, "tflops": info["flops"] / ms / 1e9, "splits": info["splits"]}
    for name, rows in (("hc_decode", 5), ("hc_wide", 2048)):
        if want(name) or want("hc"):
            run, info = hc_case(rows)
            ms = _time(run, args.reps)
            lib.raise_on_status(info["status"], name)
            out[name] = {"ms": ms, "rows": rows, "gb_s": info["bytes_min"] / ms / 1e6,
                         "kernels": "hc_step" if rows <= 16 else "hc_post_mix + hc_finish"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
