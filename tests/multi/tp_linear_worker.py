"""Worker: fused all-gather->GEMM and GEMM->reduce-scatter vs NCCL + library matmul, with device timings."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from ds41rt_b200.ops import lib  # noqa: E402
from ds41rt_b200.parallel.fabric import Fabric  # noqa: E402
from ds41rt_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear, SyncFlags  # noqa: E402


def timed(f, fn, reps):
    for _ in range(3):
        fn()
    f.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return f.all_reduce_max(e0.elapsed_time(e1) / reps)


def main():
    f = Fabric.create()
    rows = int(os.environ.get("TP_ROWS", "1024"))
    K, N = int(os.environ.get("TP_K", "5120")), int(os.environ.get("TP_N", "4096"))
    reps = int(os.environ.get("TP_REPS", "10"))
    W = f.world
    g = torch.Generator(device=f.device).manual_seed(100 + f.rank)
    flags = SyncFlags(f)
    # ---- all-gather -> GEMM (q_b / shared-up shape): x sharded by rows, weights sharded by output columns
    col = ColumnParallelLinear(f, (torch.randn(N // W, K, device=f.device, generator=g) * 0.05).bfloat16(), rows, flags)
    out = torch.zeros(W * rows, N // W, dtype=torch.bfloat16, device=f.device)
    ref = torch.zeros_like(out)
    for it in range(3):                                    # repeated calls exercise the alternating buffers
        xs = torch.randn(rows, K, device=f.device, generator=g).bfloat16()
        col.x.copy_(xs)
        keep = col.x
        col.baseline(ref)
        col.forward(out)
        torch.cuda.synchronize()
        lib.raise_on_status(flags.status, "ag_gemm")
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert err < 2e-2, ("ag_gemm", it, err)
    t_ag = timed(f, lambda: col.forward(out), reps)
    t_ag_base = timed(f, lambda: col.baseline(ref), reps)
    # ---- GEMM -> reduce-scatter (o_b / shared-down shape): K sharded, output rows scattered
    row = RowParallelLinear(f, (torch.randn(K, N // W, device=f.device, generator=g) * 0.05).bfloat16(), rows, flags)
    y = torch.zeros(rows, K, dtype=torch.bfloat16, device=f.device)
    yref = torch.zeros_like(y)
    for it in range(3):
        xin = torch.randn(W * rows, N // W, device=f.device, generator=g).bfloat16()
        row.baseline(xin, yref)
        row.forward(xin, y)
        torch.cuda.synchronize()
        lib.raise_on_status(flags.status, "gemm_rs")
        err = float((y.float() - yref.float()).abs().max() / yref.float().abs().max())
        assert err < 2e-2, ("gemm_rs", it, err)
    t_rs = timed(f, lambda: row.forward(xin, y), reps)
    t_rs_base = timed(f, lambda: row.baseline(xin, yref), reps)
    if f.rank == 0:
        flops = 2.0 * W * rows * K * (N // W)
        link = 770e9
        ag_bytes = (W - 1) * rows * K * 2                  # bytes this GPU pushes over NVLink (bf16 rows)
        rs_bytes = (W - 1) * rows * K * 2                  # bf16 partial rows pushed to the peers
        peak = float(os.environ.get("PEAK_TFLOPS", "1430")) * 1e12
        res = {"world": W, "rows_per_rank": rows, "K": K, "N": N,
               "ag_gemm_ms": t_ag, "ag_gemm_nccl_ms": t_ag_base, "gemm_rs_ms": t_rs, "gemm_rs_nccl_ms": t_rs_base,
               "ag_roofline_ms": max(flops / peak, ag_bytes / link) * 1e3,
               "rs_roofline_ms": max(flops / peak, rs_bytes / link) * 1e3}
        res["ag_frac_of_roofline"] = res["ag_roofline_ms"] / t_ag
        res["rs_frac_of_roofline"] = res["rs_roofline_ms"] / t_rs
        print("TP_LINEAR " + json.dumps(res))
        print("TP_LINEAR_OK")
    f.barrier()


if __name__ == "__main__":
    main()
