"""Same-box timing arms that run the reference's own CUDA kernels through its stock C entry points.

`baseline/build_ref.py` links the reference's unmodified `native/cuda/kernels/*.cu` objects into
`baseline/_ref/libds41rt_ref_kernels.so`; this module loads that library with ctypes and builds, for each kernel, inputs
that satisfy the contract written in the reference's headers (every launcher validates spans, alignment and disjointness
on the host and returns an error code before it launches anything):

  attention   ds41rt_v41_sparse_attention / _split      native/include/ds41rt_v41_sparse_attention.h:24-68
  topk        ds41rt_v41_index_top512                    native/include/ds41rt_v41_index_topk.h:6-19
  router      ds41rt_v41_router                          native/include/ds41rt_v41_router.h:6-14
  hc          ds41rt_v41_hc_post + _mixes + _pre         native/include/ds41rt_v41_hc.h:6-20
  index       ds41rt_v41_index_scores                    native/include/ds41rt_v41_index_scores.h:10-22
  sampler     ds41rt_cuda_v41_target_sample_async + _topk_select_async + _nucleus_async (K1/K2, K3/K4, K5)
                                                         native/cuda/kernels/v41_sampling_gpu.h:286-420

The shapes are those of `kernel_case` (window 128 + 512 selected keys, 64 heads x 512, FP8 window rows and FP4
compressed rows; 384 experts over a 5120-wide hidden row; 4 residual streams).  Each case returns a closure that
launches the reference kernel(s) once on the current stream, and a dict describing the work.  None of this package's
kernels runs on this path.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

_LIB: Optional[C.CDLL] = None
_WHY = ""


def library_path() -> str:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    return os.path.join(root, "baseline", "_ref", "libds41rt_ref_kernels.so")


def library() -> Optional[C.CDLL]:
    """The reference kernel library, or None (then `why()` says what is missing)."""
    global _LIB, _WHY
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.isfile(path):
        _WHY = "baseline/_ref/libds41rt_ref_kernels.so is not built (python baseline/build_ref.py --source <tree>)"
        return None
    try:
        _LIB = C.CDLL(path)
    except OSError as exc:
        _WHY = f"cannot load the reference kernel library: {exc}"
        return None
    for name in ("ds41rt_cuda_v41_target_sample_async", "ds41rt_cuda_v41_topk_select_async",
                 "ds41rt_cuda_v41_nucleus_async"):
        getattr(_LIB, name).restype = C.c_int32
    for name in ("ds41rt_v41_sparse_attention", "ds41rt_v41_sparse_attention_split", "ds41rt_v41_index_top512",
                 "ds41rt_v41_router", "ds41rt_v41_hc_pre", "ds41rt_v41_hc_post", "ds41rt_v41_hc_mixes",
                 "ds41rt_v41_index_scores", "ds41rt_v41_sparse_attention_initialize", "ds41rt_v41_router_initialize"):
        getattr(_LIB, name).restype = C.c_int32
    return _LIB


def why() -> str:
    return _WHY


class SparseKv(C.Structure):
    """ds41rt_v41_sparse_kv_t (native/include/ds41rt_v41_sparse_attention.h:9-22)."""
    _fields_ = [("values", C.c_void_p * 4), ("scales", C.c_void_p * 4), ("window_end", C.c_void_p),
                ("pages", C.c_void_p), ("source_end", C.c_void_p), ("window_proposal_capacity", C.c_uint64),
                ("source_capacity", C.c_uint64), ("source_proposal_capacity", C.c_uint64), ("page_stride", C.c_uint32),
                ("compressed", C.c_uint32)]


def _p(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"reference {what} returned {code}")


def attention_case(rows: int, ctx: int = 16384, check_rows: int = 0):
    """`rows` consecutive query positions ending at `ctx`: the last committed position is ctx - rows, so each row's
    128-key window mixes ring rows (committed) with rows of the private window wave; 512 selected rows of a paged FP4
    pool follow.  rows <= 64 takes the split entry point with 10 key partitions (the reference's decode form)."""
    from ..ops import quant_ref as Q
    lib = library()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    heads, D, topk = 64, 512, 512
    p0 = ctx - rows
    n_comp = ctx // 4
    ring = torch.randn(128, D, device=dev, generator=g)
    wave = torch.randn(rows, D, device=dev, generator=g)
    pool = torch.randn(n_comp, D, device=dev, generator=g)
    rq, re = Q.quant_mxfp8(ring, 32)
    wq, we = Q.quant_mxfp8(wave, 32)
    pq, ps = Q.quant_kv_fp4_e4m3_16(pool)
    ring_v, ring_s = rq.view(torch.uint8).contiguous(), re.to(torch.uint8).contiguous()
    wave_v, wave_s = wq.view(torch.uint8).contiguous(), we.to(torch.uint8).contiguous()
    pool_v = pq.view(torch.uint8).reshape(n_comp, D // 2).contiguous()
    pool_s = ps.view(torch.uint8).reshape(n_comp, D // 16).contiguous()
    spare_v = torch.zeros(256, dtype=torch.uint8, device=dev)          # one unused private source row
    spare_s = torch.zeros(32, dtype=torch.uint8, device=dev)
    window_end = torch.tensor([p0], dtype=torch.int64, device=dev)
    source_end = torch.tensor([n_comp], dtype=torch.int64, device=dev)
    n_pages = (n_comp + 255) // 256
    pages = torch.arange(n_pages, dtype=torch.int32, device=dev)
    meta = torch.zeros(rows, 10, dtype=torch.int64, device=dev)
    meta[:, 0], meta[:, 1], meta[:, 2] = p0, 0, rows
    meta[:, 3] = torch.arange(p0, p0 + rows, device=dev)
    meta[:, 5], meta[:, 6], meta[:, 9] = n_comp - 8, n_comp, 1
    sel = torch.stack([torch.sort(torch.randperm(n_comp - 8, device=dev, generator=g)[:topk]).values
                       for _ in range(rows)]).int().contiguous()
    q = torch.randn(rows, heads, D, device=dev, generator=g).bfloat16()
    sink = torch.zeros(heads, device=dev)
    out = torch.zeros(rows, heads, D, device=dev, dtype=torch.bfloat16)
    view = SparseKv()
    for i, (v, s) in enumerate(((ring_v, ring_s), (wave_v, wave_s), (pool_v, pool_s), (spare_v, spare_s))):
        view.values[i], view.scales[i] = v.data_ptr(), s.data_ptr()
    view.window_end, view.pages, view.source_end = window_end.data_ptr(), pages.data_ptr(), source_end.data_ptr()
    view.window_proposal_capacity, view.source_capacity, view.source_proposal_capacity = rows, n_comp, 1
    view.page_stride, view.compressed = n_pages, 2
    _check(lib.ds41rt_v41_sparse_attention_initialize(), "sparse_attention_initialize")
    parts = 10 if rows <= 64 else 1
    partial = torch.zeros(rows * parts * heads * 514, device=dev) if parts > 1 else None
    keep = (ring_v, ring_s, wave_v, wave_s, pool_v, pool_s, spare_v, spare_s, window_end, source_end, pages, meta, sel,
            q, sink, out, partial)

    def run():
        if parts > 1:
            _check(lib.ds41rt_v41_sparse_attention_split(_p(q), _p(sink), _p(meta), _p(sel), _p(out), rows, 128,
                                                         C.byref(view), _stream(), _p(partial),
                                                         C.c_uint64(partial.numel() * 4), parts), "sparse_attention_split")
        else:
            _check(lib.ds41rt_v41_sparse_attention(_p(q), _p(sink), _p(meta), _p(sel), _p(out), rows, 128,
                                                   C.byref(view), _stream()), "sparse_attention")
    info = {"rows": rows, "keys_per_row": 128 + topk, "flops": 2.0 * 2.0 * rows * heads * (128 + topk) * D, "keep": keep,
            "entry": "ds41rt_v41_sparse_attention_split (10 parts)" if parts > 1 else "ds41rt_v41_sparse_attention"}
    if check_rows:
        run()
        torch.cuda.synchronize()
        ring_f = Q.dequant_mxfp8(rq, re, 32).bfloat16().float()
        wave_f = Q.dequant_mxfp8(wq, we, 32).bfloat16().float()
        pool_f = Q.dequant_kv_fp4_e4m3_16(pq, ps).reshape(n_comp, D).bfloat16().float()
        worst = 0.0
        for r in list(range(min(check_rows, rows))) + [rows - 1]:
            pos = p0 + r
            keys = [ring_f[p % 128] if p < p0 else wave_f[p - p0] for p in range(pos - 127, pos + 1)]
            keys = torch.cat([torch.stack(keys), pool_f[sel[r].long()]])
            s = (q[r].float() @ keys.T) * D ** -0.5
            m = s.amax(-1, keepdim=True).clamp_min(0)
            e = torch.exp(s - m)
            want = (e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None] - m))) @ keys
            worst = max(worst, float((out[r].float() - want).abs().max() / want.abs().max()))
        info["max_rel_err_vs_fp32"] = worst
    return run, info


def topk_case(queries: int = 1024, candidates: int = 16384):
    lib = library()
    dev = torch.device("cuda")
    scores = torch.randn(queries, candidates, device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    positions = torch.arange(candidates, dtype=torch.int64, device=dev).repeat(queries, 1).contiguous()
    carry = torch.zeros(queries, 512, dtype=torch.int64, device=dev)
    scratch_bytes = queries * ((candidates + 1023) // 1024) * 512 * 8 * 2
    scratch = torch.zeros(scratch_bytes, dtype=torch.uint8, device=dev)
    out = torch.zeros(queries, 512, dtype=torch.int32, device=dev)

    def run():
        _check(lib.ds41rt_v41_index_top512(_p(scores), _p(positions), _p(carry), _p(scratch), C.c_uint64(scratch_bytes),
                                           _p(out), queries, candidates, 1, _stream()), "index_top512")
    return run, {"bytes_min": 4.0 * queries * candidates, "keep": (scores, positions, carry, scratch, out),
                 "scores": scores, "out": out}


def router_case(rows: int, experts: int = 384, H: int = 5120):
    """Hidden rows x gate weight -> sqrt-softplus scores -> top 6 with normalised weights, as one entry point."""
    lib = library()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    hidden = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    weight = (torch.randn(experts, H, device=dev, generator=g) * H ** -0.5).bfloat16()
    bias = torch.randn(experts, device=dev, generator=g) * 0.01
    scores = torch.zeros(rows, experts, device=dev)
    ids = torch.zeros(rows, 6, dtype=torch.int32, device=dev)
    routing = torch.zeros(rows, 6, device=dev)
    _check(lib.ds41rt_v41_router_initialize(), "router_initialize")

    def run():
        _check(lib.ds41rt_v41_router(_p(hidden), _p(weight), _p(bias), _p(None), _p(None), _p(scores), _p(ids),
                                     _p(routing), rows, experts, _stream()), "router")
    return run, {"rows": rows, "flops": 2.0 * rows * experts * H, "keep": (hidden, weight, bias, scores, ids, routing),
                 "hidden": hidden, "weight": weight, "bias": bias, "ids": ids, "routing": routing}


def hc_case(rows: int, H: int = 5120):
    """One sublayer boundary of the 4-stream hyper-connection: expand with the sublayer output (post), the next
    sublayer's mixes (project + Sinkhorn), and the collapse to one row (pre).  The reference's RMSNorm is a separate
    kernel and is not part of this arm."""
    lib = library()
    assert H == 5120
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    residual = torch.randn(rows, 4, H, device=dev, generator=g).bfloat16()
    sublayer = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    fn = torch.randn(24, 4 * H, device=dev, generator=g) * 0.02
    scale = torch.tensor([1.0, 0.7, 1.3], device=dev)
    base = torch.randn(24, device=dev, generator=g) * 0.5
    post = torch.rand(rows, 4, device=dev, generator=g)
    comb = torch.rand(rows, 16, device=dev, generator=g)
    expanded = torch.zeros_like(residual)
    pre = torch.zeros(rows, 4, device=dev)
    post2 = torch.zeros(rows, 4, device=dev)
    comb2 = torch.zeros(rows, 16, device=dev)
    collapsed = torch.zeros(rows, H, device=dev, dtype=torch.bfloat16)

    def run():
        s = _stream()
        _check(lib.ds41rt_v41_hc_post(_p(sublayer), _p(residual), _p(post), _p(comb), _p(expanded), rows, s), "hc_post")
        _check(lib.ds41rt_v41_hc_mixes(_p(expanded), _p(fn), _p(scale), _p(base), _p(pre), _p(post2), _p(comb2), rows, s),
               "hc_mixes")
        _check(lib.ds41rt_v41_hc_pre(_p(expanded), _p(pre), _p(collapsed), rows, s), "hc_pre")
    streams_bytes = 2.0 * rows * 4 * H
    return run, {"rows": rows, "bytes_min": 2 * streams_bytes + 2.0 * rows * H * 2 + 4.0 * 24 * 4 * H,
                 "keep": (residual, sublayer, fn, scale, base, post, comb, expanded, pre, post2, comb2, collapsed)}


def index_case(queries: int = 256, candidates: int = 16384):
    """Lightning-indexer scores: 32 heads x 128 dims, FP4 queries and keys with one E8M0 scale per 32 values."""
    lib = library()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(4)
    rb = lambda *shape, hi=256: torch.randint(0, hi, shape, dtype=torch.uint8, device=dev, generator=g)
    q, keys = rb(queries, 32 * 64), rb(candidates, 64)
    qs = (torch.randint(120, 130, (queries, 128), device=dev, generator=g)).to(torch.uint8)
    ks = (torch.randint(120, 130, (candidates, 4), device=dev, generator=g)).to(torch.uint8)
    weights = torch.rand(queries, 32, device=dev, generator=g).bfloat16()
    stride = (candidates + 255) // 256
    pages = torch.arange(stride, dtype=torch.int32, device=dev)
    lengths = torch.tensor([candidates], dtype=torch.int64, device=dev)
    meta = torch.zeros(queries, 2, dtype=torch.int64, device=dev)
    meta[:, 1] = candidates
    positions = torch.arange(candidates, dtype=torch.int64, device=dev).repeat(queries, 1).contiguous()
    out = torch.zeros(queries, candidates, device=dev)

    def run():
        _check(lib.ds41rt_v41_index_scores(_p(q), _p(qs), _p(weights), _p(keys), _p(ks), _p(pages), _p(lengths), _p(meta),
                                           _p(positions), _p(out), queries, candidates, 1, stride,
                                           C.c_uint64(candidates), _stream()), "index_scores")
    return run, {"flops": 2.0 * queries * 32 * candidates * 128, "queries": queries, "candidates": candidates,
                 "keep": (q, qs, weights, keys, ks, pages, lengths, meta, positions, out), "out": out}


def sampler_case(rows: int = 8, vocab: int = 129280, top_k: int = 50, top_p: float = 0.9, temperature: float = 0.8):
    """The reference's GPU target sampler for `rows` unconstrained rows: K1 (mask / finiteness / scaled maximum) + K2, then
    K3 / K4 (exact top-k membership in rank order), then K5 (top-p nucleus and the (seed, position) draw).  Row r uses
    seed r and position 0, as the `sampler` case of kernel_case does."""
    import numpy as np
    lib = library()
    dev = torch.device("cuda")
    logits = torch.randn(rows, vocab, device=dev, generator=torch.Generator(device=dev).manual_seed(3)) * 3
    row_t = np.dtype([("seed", "<u8"), ("position", "<u8"), ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"),
                      ("top_k", "<u4"), ("mask_row", "<u4"), ("flags", "<u4"), ("output_row", "<u4"), ("ln_min_p", "<f4"),
                      ("reserved0", "<u4"), ("reserved1", "<u4"), ("reserved2", "<u8")])
    assert row_t.itemsize == 64
    host = np.zeros(rows, dtype=row_t)
    host["seed"], host["position"] = np.arange(rows), 0
    host["temperature"], host["top_p"], host["min_p"], host["top_k"] = temperature, top_p, 0.0, top_k
    host["mask_row"], host["flags"], host["output_row"] = 0xFFFFFFFF, 0x4, np.arange(rows)     # unconstrained rows
    host["ln_min_p"] = -np.inf
    params = torch.from_numpy(host.view(np.uint8).reshape(rows, 64).copy()).to(dev)
    u32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
    f32 = lambda n: torch.zeros(n, dtype=torch.float32, device=dev)
    out_idx, out_status, out_detail, retained, passes, nucleus = u32(rows), u32(rows), u32(rows), u32(rows), u32(rows), u32(rows)
    out_scores, out_total = f32(rows), f32(rows)
    scratch = torch.zeros(rows * 64, dtype=torch.uint8, device=dev)
    cap = 256
    assert top_k <= cap
    rank_ids = u32(rows * cap)
    rank_scratch = torch.zeros(rows * cap, dtype=torch.int64, device=dev)
    z = C.c_size_t

    def run():
        s = _stream()
        _check(lib.ds41rt_cuda_v41_target_sample_async(_p(logits), z(rows), z(vocab), z(vocab), _p(params), _p(None), z(0),
                                                       _p(out_idx), _p(out_status), _p(out_detail), _p(out_scores),
                                                       _p(out_total), _p(nucleus), _p(scratch), s), "target_sample")
        _check(lib.ds41rt_cuda_v41_topk_select_async(_p(logits), z(rows), z(vocab), z(vocab), _p(params), _p(None), z(0),
                                                     _p(rank_ids), _p(rank_scratch), z(cap), _p(retained), _p(passes),
                                                     _p(scratch), s), "topk_select")
        _check(lib.ds41rt_cuda_v41_nucleus_async(_p(logits), z(rows), z(vocab), z(vocab), _p(params), _p(None), z(0),
                                                 _p(rank_ids), z(cap), _p(retained), _p(out_idx), _p(out_status),
                                                 _p(out_total), _p(nucleus), _p(scratch), s), "nucleus")
    return run, {"bytes_min": 4.0 * rows * vocab, "logits": logits, "tokens": out_idx, "status": out_status,
                 "keep": (params, out_detail, retained, passes, nucleus, out_scores, out_total, scratch, rank_ids,
                          rank_scratch)}
