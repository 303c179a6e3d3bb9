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
    cases = [("bf16_gemm_%d" % n, big, 2.0 * n ** 3, None), ("decode_head_shard", skinny, None, V * H * 2),
             ("mxfp8_expert_fc1", fc1, None, 6 * 2 * I * H), ("mxfp4_expert_fc1", fc1_fp4, None, 6 * 2 * I * H // 2),
             ("nvfp4_expert_fc1", fc1_nv, None, 6 * 2 * I * H // 2)]
    for name, fn, flops, nbytes in cases:
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
