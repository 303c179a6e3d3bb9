"""Stand-alone GEMM cases for timing and profiling the tcgen05 kernel.

    python -m ds41rt_b200.utils.gemm_case            # times every case, prints achieved TFLOP/s or GB/s
    python -m ds41rt_b200.utils.gemm_case --once     # one launch per case after warm-up (profiler captures)
Cases: a compute-bound bf16 GEMM (operands larger than L2), a bandwidth-bound decode projection (8 rows against a
vocabulary shard, swap-AB) and the block-scaled FP8 expert FC1 (dual gate/up tiles, SwiGLU epilogue).
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import gemm as G
from ..ops import lib


def _time(fn, reps):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--only", default="", help="comma-separated case names (default: all)")
    args = ap.parse_args()
    dev = "cuda"
    st = lib.new_status(dev)
    out = {}
    # ---- compute bound
    n = args.size
    x = torch.randn(n, n, device=dev).bfloat16()
    w = torch.randn(n, n, device=dev).bfloat16()
    y = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
    big = lambda: G.gemm_raw(x, w, y, n, n, n, lda=n, ldb=n, ldo=n, out_mode=6, bn=256, status=st, static_operand=2)
    # ---- bandwidth bound (decode head shard)
    rows, V, H = 8, 16160, 5120
    xs = torch.randn(rows, H, device=dev).bfloat16()
    wh = torch.randn(V, H, device=dev).bfloat16()
    lg = torch.empty(rows, V, device=dev)
    skinny = lambda: G.gemm_raw(wh, xs, lg, V, rows, H, lda=H, ldb=H, ldo=V, out_mode=3, status=st, static_operand=1)
    # ---- block-scaled FP8 expert FC1 (6 active experts, 8 rows)
    E, I = 8, 2304
    w13 = (torch.randn(E, 2 * I, H, device=dev) * 48).clamp(-448, 448).to(torch.float8_e4m3fn)
    w13_sf = torch.full((E, 2 * I // 128, H // 128, 512), 116, dtype=torch.uint8, device=dev)
    xq = torch.randn(rows, H, device=dev).to(torch.float8_e4m3fn)
    xq_sf = torch.full((1, H // 128, 512), 127, dtype=torch.uint8, device=dev)
    act = torch.zeros(6, rows, I, device=dev, dtype=torch.bfloat16)
    active = torch.arange(6, dtype=torch.int32, device=dev)
    n_active = torch.tensor([6], dtype=torch.int32, device=dev)
    row_w = torch.ones(6, rows, device=dev)
    fc1 = lambda: G.gemm_raw(w13, xq, act, I, rows, H, lda=H, ldb=H, ldo=I, kind=2, out_mode=4, bn=16, batch=6,
                             a_batches=E, a_batch_stride=2 * I * H, out_batch_stride=rows * I, batch_map=active,
                             n_active=n_active, b_batch_kind=1, up_row_offset=I, row_w=row_w, row_w_ld=rows,
                             sfa=w13_sf, sfa_batch_stride=w13_sf[0].numel(), sfb=xq_sf, status=st)
    w13_4 = torch.randint(0, 256, (E, 2 * I, H // 2), dtype=torch.uint8, device=dev)
    fc1_fp4 = lambda: G.gemm_raw(w13_4, xq, act, I, rows, H, lda=H, ldb=H, ldo=I, kind=2, out_mode=4, bn=16, batch=6,
                                 a_batches=E, a_batch_stride=2 * I * H, out_batch_stride=rows * I, batch_map=active,
                                 n_active=n_active, b_batch_kind=1, up_row_offset=I, row_w=row_w, row_w_ld=rows,
                                 sfa=w13_sf, sfa_batch_stride=w13_sf[0].numel(), sfb=xq_sf, status=st, a_format=1)
    # NVFP4 W4A4: both operands e2m1, E4M3 scale per 16, 64 K elements per instruction
    xq4 = torch.randint(0, 256, (rows, H // 2), dtype=torch.uint8, device=dev)
    xq4_sf = torch.full((1, H // 64, 512), 0x38, dtype=torch.uint8, device=dev)
    w13_sf4 = torch.full((E, 2 * I // 128, H // 64, 512), 0x38, dtype=torch.uint8, device=dev)
    fc1_nv = lambda: G.gemm_raw(w13_4, xq4, act, I, rows, H, lda=H, ldb=H, ldo=I, kind=3, out_mode=4, bn=32, batch=6,
                                a_batches=E, a_batch_stride=2 * I * H, out_batch_stride=rows * I, batch_map=active,
                                n_active=n_active, b_batch_kind=1, up_row_offset=I, row_w=row_w, row_w_ld=rows,
                                sfa=w13_sf4, sfa_batch_stride=w13_sf4[0].numel(), sfb=xq4_sf, status=st, alpha=0.01)
    # ---- a verification pass's expert layer: 5 rows that reach 30 of 40 resident experts (block-scaled FP8), FC1 and FC2
    # through the active-expert list exactly as the engine launches them (grid sized for the worst case, a device count)
    E2, act_n, r5, cap = 40, 30, 5, 64
    w13b = (torch.randn(E2, 2 * I, H, device=dev) * 48).clamp(-448, 448).to(torch.float8_e4m3fn)
    w13b_sf = torch.full((E2, 2 * I // 128, H // 128, 512), 116, dtype=torch.uint8, device=dev)
    w2b = (torch.randn(E2, H, I, device=dev) * 48).clamp(-448, 448).to(torch.float8_e4m3fn)
    w2b_sf = torch.full((E2, H // 128, I // 128, 512), 116, dtype=torch.uint8, device=dev)
    x5 = torch.randn(r5, H, device=dev).to(torch.float8_e4m3fn)
    actb = torch.zeros(cap, r5, I, device=dev, dtype=torch.bfloat16)
    actq = torch.randn(cap, r5, I, device=dev).to(torch.float8_e4m3fn)
    actq_sf = torch.full((cap, 1, I // 128, 512), 127, dtype=torch.uint8, device=dev)
    fc2_out = torch.zeros(cap, r5, H, device=dev)
    active2 = torch.arange(cap, dtype=torch.int32, device=dev) % E2
    n_active2 = torch.tensor([act_n], dtype=torch.int32, device=dev)
    row_w2 = torch.ones(cap, 32, device=dev)
    fc1_30 = lambda: G.gemm_raw(w13b, x5, actb, I, r5, H, lda=H, ldb=H, ldo=I, kind=2, out_mode=4, bn=16, batch=cap,
                                a_batches=E2, a_batch_stride=2 * I * H, out_batch_stride=r5 * I, batch_map=active2,
                                n_active=n_active2, b_batch_kind=1, up_row_offset=I, row_w=row_w2, row_w_ld=32,
                                sfa=w13b_sf, sfa_batch_stride=w13b_sf[0].numel(), sfb=xq_sf, status=st)
    fc2_30 = lambda: G.gemm_raw(w2b, actq, fc2_out, H, r5, I, lda=I, ldb=I, ldo=H, kind=2, out_mode=5, bn=16, batch=cap,
                                a_batches=E2, a_batch_stride=H * I, b_batch_stride=r5 * I, out_batch_stride=r5 * H,
                                batch_map=active2, n_active=n_active2, b_batch_kind=2, row_w=row_w2, row_w_ld=32,
                                sfa=w2b_sf, sfa_batch_stride=w2b_sf[0].numel(), sfb=actq_sf,
                                sfb_batch_stride=actq_sf[0].numel(), status=st)
    cases = [("mxfp8_expert_fc1_30_experts", fc1_30, None, act_n * 2 * I * H),
             ("mxfp8_expert_fc2_30_experts", fc2_30, None, act_n * I * H),
             ("bf16_gemm_%d" % n, big, 2.0 * n ** 3, None), ("decode_head_shard", skinny, None, V * H * 2),
             ("mxfp8_expert_fc1", fc1, None, 6 * 2 * I * H), ("mxfp4_expert_fc1", fc1_fp4, None, 6 * 2 * I * H // 2),
             ("nvfp4_expert_fc1", fc1_nv, None, 6 * 2 * I * H // 2)]
    only = set(filter(None, args.only.split(",")))
    for name, fn, flops, nbytes in cases:
        if only and name not in only:
            continue
        if args.once:
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            fn()
            torch.cuda.synchronize()
            continue
        ms = _time(fn, args.reps)
        out[name] = {"ms": ms}
        if flops:
            out[name]["tflops"] = flops / ms / 1e9
        if nbytes:
            out[name]["gb_s"] = nbytes / ms / 1e6
    lib.raise_on_status(st, "gemm cases")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
