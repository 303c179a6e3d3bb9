"""Worker: fused expert-parallel layer (P2P dispatch, grouped tcgen05 GEMMs, P2P combine) vs NCCL all-to-all +
library matmuls, with device timings (max over ranks).  Runs at any world size, 1 included."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from ds41rt_b200.parallel.ep import ExpertParallelMoE  # noqa: E402
from ds41rt_b200.parallel.fabric import Fabric  # noqa: E402


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


def make_routes(T, E, topk, skew, gen, device):
    """topk distinct experts per token; with skew, two experts draw a quarter of all routes."""
    score = torch.rand(T, E, device=device, generator=gen)
    if skew:
        score[:, :2] += 0.75 * (torch.rand(T, 2, device=device, generator=gen) < 0.75)
    ids = score.topk(topk, dim=1).indices.int()
    w = torch.rand(T, topk, device=device, generator=gen) + 0.1
    return ids.contiguous(), (w / w.sum(1, keepdim=True) * 1.5).float().contiguous()


def main():
    f = Fabric.create()
    W, dev = f.world, f.device
    T = int(os.environ.get("EP_TOKENS", "512"))
    H, I = int(os.environ.get("EP_H", "1024")), int(os.environ.get("EP_I", "512"))
    E, topk = int(os.environ.get("EP_E", "16")), int(os.environ.get("EP_TOPK", "4"))
    reps, skew = int(os.environ.get("EP_REPS", "5")), int(os.environ.get("EP_SKEW", "0"))
    mx = int(os.environ.get("EP_MX", "0"))
    wire = os.environ.get("EP_WIRE", "auto")       # block-scaled experts: "fp8" (sender quantises) or "bf16" rows on NVLink
    EL = E // W
    g = torch.Generator(device=dev).manual_seed(7 + f.rank)
    w13 = (torch.randn(EL, 2 * I, H, device=dev, generator=g) * 0.04)
    w2 = (torch.randn(EL, H, I, device=dev, generator=g) * 0.04)
    if mx:
        from ds41rt_b200.models.ds41 import dequantize_expert, quantize_expert_stack
        q13, s13 = quantize_expert_stack(w13.cpu(), dev)
        q2, s2 = quantize_expert_stack(w2.cpu(), dev)
        moe = ExpertParallelMoE(f, q13, q2, topk=topk, max_tokens=T, w13_sf=s13, w2_sf=s2, wire=wire,
                                tile_tokens=int(os.environ["EP_TILE"]) if os.environ.get("EP_TILE") else None)
        w13_ref = torch.stack([dequantize_expert(q13[e], s13[e]) for e in range(EL)]).to(dev).bfloat16()
        w2_ref = torch.stack([dequantize_expert(q2[e], s2[e]) for e in range(EL)]).to(dev).bfloat16()
    else:
        w13_ref, w2_ref = w13.bfloat16(), w2.bfloat16()
        moe = ExpertParallelMoE(f, w13_ref, w2_ref, topk=topk, max_tokens=T)
    out = torch.zeros(T, H, dtype=torch.float32, device=dev)
    tol = 6e-2 if mx else 2e-2
    for it in range(3):
        x = torch.randn(T, H, device=dev, generator=g).bfloat16()
        ids, wts = make_routes(T, E, topk, skew or it == 2, g, dev)
        if it == 1:
            ids[::7, 0] = -1                       # dropped routes contribute nothing
        extra = torch.randn(T, H, device=dev, generator=g) if it == 1 else None
        ref = moe.baseline(x, ids, wts, w13_ref, w2_ref, extra)
        moe.forward(x, ids, wts, out, extra)
        torch.cuda.synchronize()
        moe.check()
        err = float((out - ref).abs().max() / ref.abs().max())
        assert err < tol, ("ep", it, err)
        first = out.clone()
        moe.forward(x, ids, wts, out, extra)
        torch.cuda.synchronize()
        assert torch.equal(first, out), "expert-parallel layer is not bit-reproducible"
    t_fused = timed(f, lambda: moe.forward(x, ids, wts, out, extra), reps)
    t_base = timed(f, lambda: moe.baseline(x, ids, wts, w13_ref, w2_ref, extra), reps)
    moe.check()
    phases = moe.phase_times(x, ids, wts, out, extra, reps=reps) if int(os.environ.get("EP_PHASES", "0")) else None
    if f.rank == 0:
        routes = T * topk                                       # per rank
        flops = 2.0 * routes * H * (3 * I)                      # per rank when balanced
        peak = float(os.environ.get("PEAK_TFLOPS", "1430")) * 1e12 * (2 if mx else 1)
        link = 770e9
        remote = routes * (W - 1) / W
        out_row = (H + H // 32) if (mx and wire != "bf16") else 2 * H     # FP8 + scales on the way out, bf16 back
        nv_bytes = remote * (out_row + H * 2)
        res = {"world": W, "tokens_per_rank": T, "H": H, "I": I, "E": E, "topk": topk, "skew": skew, "mx": mx,
               "wire": ("fp8" if (mx and wire != "bf16") else "bf16"),
               "fused_ms": t_fused, "nccl_library_ms": t_base,
               "roofline_ms": max(flops / peak, (nv_bytes / 2) / link) * 1e3}
        res["frac_of_roofline"] = res["roofline_ms"] / t_fused
        if phases:
            res["phases_ms_rank0"] = {k: round(v, 4) for k, v in phases.items()}
        print("EP " + json.dumps(res))
        print("EP_OK")
    f.barrier()


if __name__ == "__main__":
    main()
