"""Individual CUDA kernels vs plain PyTorch fp32 references of the same op."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("max_keys,positions", [(5000, [4999, 2999, 300, 4000]),        # register forms (8 / 4 keys a thread)
                                                (20000, [15999, 19999, 2047, 9000]),    # 16 a thread; streaming form
                                                (1024, [1023, 700, 511, 600])])
def test_topk_select_exact(max_keys, positions):
    from ds41rt_b200.ops import lib
    k = lib.kernels()
    rows, topk = 4, 512
    torch.manual_seed(0)
    scores = torch.randn(rows, max_keys, device="cuda")
    scores[1, :3000] = scores[1, :3000].round()            # many ties
    scores[0, 17] = float("-inf")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slot = torch.tensor([0, 0, 0, -1], dtype=torch.int32, device="cuda")
    sel = torch.zeros(rows, topk, dtype=torch.int32, device="cuda")
    n_sel = torch.zeros(rows, dtype=torch.int32, device="cuda")
    lib.check(k.ds41_topk_select(lib.ptr(scores), max_keys, lib.ptr(pos), lib.ptr(slot), 1, topk, lib.ptr(sel),
                                 lib.ptr(n_sel), rows, lib.stream()), "topk")
    torch.cuda.synchronize()
    for r in range(3):
        n = int(pos[r]) + 1
        got = sel[r, : int(n_sel[r])].tolist()
        if n <= topk:
            assert got == list(range(n))
            continue
        s = scores[r, :n].cpu()
        order = torch.sort(s, descending=True, stable=True).indices[:topk]
        assert got == sorted(order.tolist())
        assert int(n_sel[r]) == topk
    assert int(n_sel[3]) == 0


def _attend_ref(q, keys, sink, scale):
    # q [H, D], keys [n, D]
    logits = (q @ keys.t()) * scale
    m = torch.maximum(logits.amax(-1, keepdim=True), sink[:, None])
    e = torch.exp(logits - m)
    return (e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None] - m))) @ keys


def _pack_fp8_rows(x, row_bytes):
    """bf16 rows -> (FP8 cache rows [.., row_bytes] uint8, the dequantised values the kernel must see)."""
    from ds41rt_b200.ops import quant_ref as Q
    D = x.shape[-1]
    q, e = Q.quant_mxfp8(x.float(), 32)
    rows = torch.zeros(*x.shape[:-1], row_bytes, dtype=torch.uint8, device=x.device)
    rows[..., :D] = q.view(torch.uint8)
    rows[..., D:D + D // 32] = e.to(torch.uint8)
    return rows.contiguous(), Q.dequant_mxfp8(q, e, 32).bfloat16()


def _pack_fp4_rows(x, row_bytes):
    """bf16 rows -> (FP4 cache rows [.., row_bytes] uint8, the dequantised values the kernel must see)."""
    from ds41rt_b200.ops import quant_ref as Q
    D = x.shape[-1]
    packed, bs = Q.quant_kv_fp4_e4m3_16(x.float())
    rows = torch.zeros(*x.shape[:-1], row_bytes, dtype=torch.uint8, device=x.device)
    rows[..., :D // 2] = packed.view(torch.uint8).reshape(*x.shape[:-1], D // 2)
    rows[..., D // 2:D // 2 + D // 16] = bs.view(torch.uint8).reshape(*x.shape[:-1], D // 16)
    return rows.contiguous(), Q.dequant_kv_fp4_e4m3_16(packed, bs).reshape(x.shape).bfloat16()


@pytest.mark.parametrize("impl", ["tc", "legacy"])
@pytest.mark.parametrize("kv", ["bf16", "fp8", "fp4"])
@pytest.mark.parametrize("D,heads,rope,rows,n_splits", [(128, 8, 32, 3, 0), (512, 16, 64, 3, 0), (512, 64, 64, 3, 0),
                                                         (512, 64, 64, 70, 1), (512, 64, 64, 66, 3), (128, 64, 32, 64, 2),
                                                         (512, 64, 64, 330, 1), (512, 8, 64, 180, 2)])
def test_sparse_attention(D, heads, rope, rows, n_splits, kv, impl):
    """impl "tc": tcgen05 kernel (persistent grid over (row, key split) items, accumulators in tensor memory, final rows
    written by the kernel when there is one split); "legacy": warp-MMA kernels (rows >= 64 with 64 heads runs their wide
    form)."""
    from ds41rt_b200.ops import lib
    from ds41rt_b200.ops import attention as A
    from ds41rt_b200.config import RopeConfig, rope_inv_freq
    from ds41rt_b200.models.reference import apply_rope
    k = lib.kernels()
    torch.manual_seed(0)
    window, ring, topk, page_rows, max_pages = 128, 144 + rows, 64, 32, 16
    positions = ([700, 701, 50] + [300 + 3 * i for i in range(rows)])[:rows]
    slots = ([0, 0, 1] + [i % 2 for i in range(rows)])[:rows]
    win = torch.randn(2, ring, D, device="cuda").bfloat16()
    pool = torch.randn(max_pages * 2 * page_rows, D, device="cuda").bfloat16()
    row_bytes = 0 if kv == "bf16" else (D + D // 32 + 15) // 16 * 16      # "fp4" keeps FP8 window rows
    win_dev, pool_dev = win, pool
    comp_bytes = 0
    if row_bytes:
        win_dev, win = _pack_fp8_rows(win, row_bytes)          # the reference below sees the dequantised rows
        if kv == "fp4":                                        # FP8 window rows, FP4 compressed rows
            comp_bytes = (D // 2 + D // 16 + 15) // 16 * 16
            pool_dev, pool = _pack_fp4_rows(pool, comp_bytes)
        else:
            pool_dev, pool = _pack_fp8_rows(pool, row_bytes)
    page_table = torch.arange(2 * max_pages, dtype=torch.int32, device="cuda").view(2, max_pages).flip(1).contiguous()
    sel = torch.full((rows, topk), -1, dtype=torch.int32, device="cuda")
    counts = ([64, 40, 0] + [(7 * i) % 65 for i in range(rows)])[:rows]
    n_sel = torch.tensor(counts, dtype=torch.int32, device="cuda")
    for i, c in enumerate(counts):
        if c:
            sel[i, :c] = torch.sort(torch.randperm(300)[:c]).values.int().cuda()
    q = torch.randn(rows, heads * D, device="cuda").bfloat16()
    sink = torch.randn(heads, device="cuda")
    inv = torch.tensor(rope_inv_freq(RopeConfig(), rope), device="cuda")
    n_splits = n_splits or (window + 16 + topk + 63) // 64
    part_o = torch.zeros(rows, n_splits, heads, D, device="cuda")
    part_ml = torch.zeros(rows, n_splits, heads, 2, device="cuda")
    out = torch.zeros(rows, heads * D, device="cuda", dtype=torch.bfloat16)
    pos_t = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slot_t = torch.tensor(slots, dtype=torch.int32, device="cuda")
    scale = D ** -0.5
    status = lib.new_status(q.device)
    lib.check(A.attend(q=q, ldq=heads * D, q_off=0, rows=rows, heads=heads, D=D, window=window, ring=ring, row_pos=pos_t,
                       row_slot=slot_t, win=win_dev, comp_pool=pool_dev, sel=sel, n_sel=n_sel, k=topk,
                       page_table=page_table, max_pages=max_pages, page_rows=page_rows, inv_freq=inv, rope_dim=rope,
                       scale=scale, n_splits=n_splits, part_o=part_o, part_ml=part_ml, sink=sink, out=out,
                       ldo=heads * D, kv_row_bytes=row_bytes, comp_row_bytes=comp_bytes, status=status, impl=impl),
              "attend")
    torch.cuda.synchronize()
    lib.raise_on_status(status, "attend")
    torch.cuda.synchronize()
    for r in range(rows):
        pos, slot = positions[r], slots[r]
        lo = max(0, pos - window + 1)
        keys = [win[slot, p % ring] for p in range(lo, pos + 1)]
        for j in range(int(n_sel[r])):
            i = int(sel[r, j])
            phys = int(page_table[slot, i // page_rows]) * page_rows + i % page_rows
            keys.append(pool[phys])
        keys = torch.stack(keys).float()
        qr = apply_rope(q[r].float().view(heads, D).cpu(), torch.tensor(pos), inv.cpu(), rope).cuda()
        qr = qr.bfloat16().float()
        want = _attend_ref(qr, keys, sink, scale)
        want = apply_rope(want.cpu(), torch.tensor(pos), inv.cpu(), rope, inverse=True).cuda()
        got = out[r].float().view(heads, D)
        err = float((got - want).abs().max())
        assert err < 3e-2 * float(want.abs().max()) + 2e-3, (r, err)


def test_hc_kernels_match_oracle():
    from ds41rt_b200.ops import lib
    from ds41rt_b200.models import reference as R
    k = lib.kernels()
    torch.manual_seed(0)
    rows, H = 5, 512
    streams = torch.randn(rows, 4, H, device="cuda").bfloat16()
    sub = torch.randn(2, rows, H, device="cuda")           # two split planes
    fn = torch.randn(24, 4 * H, device="cuda") * 0.5
    scale = torch.tensor([1.0, 0.7, 1.3], device="cuda")
    base = torch.randn(24, device="cuda") * 0.5
    pre_in = torch.rand(rows, 4, device="cuda")
    norm_w = torch.rand(H, device="cuda") + 0.5
    # reference: mixes on the ORIGINAL streams give post/comb for the expand
    pre0, post0, comb0 = R.hc_mixes(streams.float().cpu(), fn.cpu(), scale.cpu(), base.cpu(), 4, 20, 1e-6, 1e-20)
    subsum = sub.sum(0).bfloat16().float().cpu()
    new_streams = R.hc_expand(streams.float().cpu(), subsum, post0, comb0).bfloat16().float()
    pre1, post1, comb1 = R.hc_mixes(new_streams, fn.cpu(), scale.cpu(), base.cpu(), 4, 20, 1e-6, 1e-20)
    xn = R.rmsnorm(R.hc_collapse(new_streams, pre_in.cpu()), norm_w.cpu(), 1e-20)
    # kernels
    st = lib.new_status("cuda")
    s_dev = streams.clone()
    partial = torch.zeros(H // 128, rows, 25, device="cuda")
    bases = (C.c_void_p * 1)(sub.data_ptr())
    post_d, comb_d = post0.cuda().contiguous(), comb0.reshape(rows, 16).cuda().contiguous()
    lib.check(k.ds41_hc_post_mix(lib.ptr(s_dev), lib.ptr(s_dev), bases, 1, 2, C.c_longlong(rows * H), lib.ptr(post_d),
                                 lib.ptr(comb_d), lib.ptr(fn), lib.ptr(partial), rows, H, lib.ptr(None), lib.ptr(None),
                                 lib.ptr(st), lib.ptr(None), lib.ptr(None), lib.ptr(None), lib.ptr(None), C.c_float(0.0), lib.stream()), "post_mix")
    next_pre = torch.zeros(rows, 4, device="cuda")
    post = torch.zeros(rows, 4, device="cuda")
    comb = torch.zeros(rows, 16, device="cuda")
    xn_d = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)
    lib.check(k.ds41_hc_finish(lib.ptr(partial), H // 128, lib.ptr(scale), lib.ptr(base), lib.ptr(pre_in),
                               lib.ptr(s_dev), lib.ptr(norm_w), lib.ptr(next_pre), lib.ptr(post), lib.ptr(comb),
                               lib.ptr(xn_d), lib.ptr(None), lib.ptr(None), lib.ptr(None), rows, H, 20, C.c_float(1e-6), C.c_float(1e-20),
                               lib.ptr(None), 0, C.c_longlong(0), 0, lib.stream()), "finish")
    torch.cuda.synchronize()
    assert (s_dev.float().cpu() - new_streams).abs().max() < 0.05
    assert (next_pre.cpu() - pre1).abs().max() < 2e-2
    assert (post.cpu() - post1).abs().max() < 2e-2
    assert (comb.cpu().view(rows, 4, 4) - comb1).abs().max() < 2e-2
    assert (xn_d.float().cpu() - xn).abs().max() < 5e-2


def test_router_select_and_plan():
    from ds41rt_b200.ops import lib
    from ds41rt_b200.models import reference as R
    k = lib.kernels()
    torch.manual_seed(0)
    rows, E, I_sh, topk = 6, 384, 64, 6
    planes = torch.randn(2, rows, E + 2 * I_sh, device="cuda")
    bias = torch.randn(E, device="cuda") * 0.01
    ids = torch.zeros(rows, topk, dtype=torch.int32, device="cuda")
    wts = torch.zeros(rows, topk, device="cuda")
    act = torch.zeros(rows, I_sh, device="cuda", dtype=torch.bfloat16)
    lib.check(k.ds41_router_select(lib.ptr(planes), 2, rows, E + 2 * I_sh, E, I_sh, topk, lib.ptr(bias),
                                   C.c_float(1.5), C.c_float(10.0), lib.ptr(ids), lib.ptr(wts), lib.ptr(act),
                                   lib.stream()), "router")
    torch.cuda.synchronize()
    logits = planes.sum(0)[:, :E].cpu()
    score = torch.sqrt(torch.nn.functional.softplus(logits))
    order = torch.sort(score + bias.cpu(), dim=-1, descending=True, stable=True).indices[:, :topk]
    sel = torch.gather(score, 1, order)
    want_w = sel / sel.sum(-1, keepdim=True) * 1.5
    assert ids.cpu().tolist() == order.tolist()
    assert (wts.cpu() - want_w).abs().max() < 1e-5
    gsum = planes.sum(0).cpu()
    want_act = R.swiglu_clamped(gsum[:, E:E + I_sh].bfloat16().float(), gsum[:, E + I_sh:].bfloat16().float(), 10.0)
    assert (act.float().cpu() - want_act).abs().max() < 2e-2
    # plan for a rank owning experts [96, 192)
    slot = torch.zeros(rows, dtype=torch.int32, device="cuda")
    max_active = 36
    active = torch.zeros(max_active, dtype=torch.int32, device="cuda")
    n_active = torch.zeros(1, dtype=torch.int32, device="cuda")
    row_w = torch.zeros(max_active, 8, device="cuda")
    slot_of = torch.zeros(rows, topk, dtype=torch.int32, device="cuda")
    lib.check(k.ds41_moe_plan(lib.ptr(ids), lib.ptr(wts), lib.ptr(slot), rows, topk, 96, 192, max_active, 8,
                              lib.ptr(active), lib.ptr(n_active), lib.ptr(row_w), lib.ptr(slot_of), lib.stream()),
              "plan")
    torch.cuda.synchronize()
    local = sorted({int(e) - 96 for e in order.flatten().tolist() if 96 <= e < 192})
    assert int(n_active) == len(local)
    assert active[: len(local)].tolist() == local
    for r in range(rows):
        for j in range(topk):
            e = int(order[r, j])
            s = int(slot_of[r, j])
            if 96 <= e < 192:
                assert local[s] == e - 96 and abs(float(row_w[s, r]) - float(want_w[r, j])) < 1e-5
            else:
                assert s == -1


@pytest.mark.parametrize("group", [32, 128])
def test_act_quant_mx(group):
    from ds41rt_b200.ops import lib, quant_ref as Q
    from ds41rt_b200.ops.mx import unpack_sf_atoms
    k = lib.kernels()
    rows, K = 37, 512
    x = (torch.randn(rows, K, device="cuda") * torch.exp(torch.randn(rows, 1, device="cuda"))).bfloat16()
    q = torch.zeros(rows, K, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(1, K // 128, 512, dtype=torch.uint8, device="cuda")
    lib.check(k.ds41_act_quant_mx(lib.ptr(x), C.c_longlong(K), C.c_longlong(0), lib.ptr(q), C.c_longlong(K),
                                  C.c_longlong(0), lib.ptr(sf), C.c_longlong(0), rows, K, 1, group, lib.ptr(None),
                                  lib.stream()), "act_quant")
    torch.cuda.synchronize()
    wq, we = Q.quant_act_fp8_ue8m0(x.float().cpu(), group)
    got_e = unpack_sf_atoms(sf.cpu(), rows)
    assert torch.equal(got_e, we)
    assert torch.equal(q.cpu().view(torch.float8_e4m3fn).float(), wq.float())


def test_hc_step_matches_unfused_kernels():
    """The fused hyper-connection step equals post_mix + finish run separately (same inputs)."""
    from ds41rt_b200.ops import lib
    k = lib.kernels()
    torch.manual_seed(1)
    rows, H = 3, 1024
    streams = torch.randn(rows, 4, H, device="cuda").bfloat16()
    sub = torch.randn(2, rows, H, device="cuda")
    fn = torch.randn(24, 4 * H, device="cuda") * 0.02
    scale = torch.tensor([1.0, 0.7, 1.3], device="cuda")
    base = torch.randn(24, device="cuda") * 0.5
    pre_in = torch.rand(rows, 4, device="cuda")
    post = torch.rand(rows, 4, device="cuda") * 2
    comb = torch.rand(rows, 16, device="cuda")
    norm_w = torch.rand(H, device="cuda") + 0.5
    st = lib.new_status("cuda")
    bases = (C.c_void_p * 1)(sub.data_ptr())
    # unfused
    s1 = streams.clone()
    partial = torch.zeros(H // 128, rows, 25, device="cuda")
    lib.check(k.ds41_hc_post_mix(lib.ptr(s1), lib.ptr(s1), bases, 1, 2, C.c_longlong(rows * H), lib.ptr(post),
                                 lib.ptr(comb), lib.ptr(fn), lib.ptr(partial), rows, H, lib.ptr(None), lib.ptr(None),
                                 lib.ptr(st), lib.ptr(None), lib.ptr(None), lib.ptr(None), lib.ptr(None), C.c_float(0.0), lib.stream()), "post_mix")
    np1, po1, co1 = torch.zeros(rows, 4, device="cuda"), torch.zeros(rows, 4, device="cuda"), torch.zeros(rows, 16, device="cuda")
    xn1 = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)
    lib.check(k.ds41_hc_finish(lib.ptr(partial), H // 128, lib.ptr(scale), lib.ptr(base), lib.ptr(pre_in),
                               lib.ptr(s1), lib.ptr(norm_w), lib.ptr(np1), lib.ptr(po1), lib.ptr(co1), lib.ptr(xn1),
                               lib.ptr(None), lib.ptr(None), lib.ptr(None), rows, H, 20, C.c_float(1e-6),
                               C.c_float(1e-20), lib.ptr(None), 0, C.c_longlong(0), 0, lib.stream()), "finish")
    # fused (run twice: the ticket counters must reset themselves)
    for _ in range(2):
        s2 = streams.clone()
        a = lib.HcStepArgs()
        np2, po2, co2 = torch.zeros(rows, 4, device="cuda"), torch.zeros(rows, 4, device="cuda"), torch.zeros(rows, 16, device="cuda")
        xn2 = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)
        xq = torch.zeros(rows, H, device="cuda", dtype=torch.uint8)
        xq_sf = torch.zeros(1, H // 128, 512, device="cuda", dtype=torch.uint8)
        if _ == 0:
            tickets = torch.zeros(rows, dtype=torch.int32, device="cuda")
        part2 = torch.zeros(H // 128, rows, 26, device="cuda")
        xc = torch.zeros(rows, H, device="cuda")
        a.streams_in = a.streams_out = lib.ptr(s2)
        a.part_bases = C.cast(bases, C.c_void_p)
        a.post, a.comb, a.pre_in = lib.ptr(post), lib.ptr(comb), lib.ptr(pre_in)
        a.fn, a.scale, a.base, a.norm_w = lib.ptr(fn), lib.ptr(scale), lib.ptr(base), lib.ptr(norm_w)
        a.partial, a.xc = lib.ptr(part2), lib.ptr(xc)
        a.next_pre, a.post_out, a.comb_out, a.xn = lib.ptr(np2), lib.ptr(po2), lib.ptr(co2), lib.ptr(xn2)
        a.xq, a.xq_sf, a.tickets, a.status = lib.ptr(xq), lib.ptr(xq_sf), lib.ptr(tickets), lib.ptr(st)
        a.split_stride, a.n_ranks, a.n_splits = rows * H, 1, 2
        a.rows, a.H, a.iters, a.hc_eps, a.norm_eps = rows, H, 20, 1e-6, 1e-20
        lib.check(k.ds41_hc_step(C.byref(a), lib.stream()), "hc_step")
        torch.cuda.synchronize()
        assert torch.equal(s1, s2)
        assert (np1 - np2).abs().max() < 1e-5 and (po1 - po2).abs().max() < 1e-5 and (co1 - co2).abs().max() < 1e-5
        assert (xn1.float() - xn2.float()).abs().max() < 2e-2
        assert int(tickets.abs().sum()) == 0
    from ds41rt_b200.ops import quant_ref as Q
    from ds41rt_b200.ops.mx import unpack_sf_atoms
    wq, we = Q.quant_act_fp8_ue8m0(xn2.float().cpu(), 128)
    assert torch.equal(unpack_sf_atoms(xq_sf.cpu(), rows), we)
    assert torch.equal(xq.cpu().view(torch.float8_e4m3fn).float(), wq.float())


def test_index_scores_on_tensor_cores_match_the_scalar_kernel():
    """One request, a long pass: RoPE'd queries x gathered keys as a GEMM with the relu / head-weight / head-sum
    epilogue gives the scores of the per-key kernel (same bf16 operands, fp32 accumulation)."""
    from ds41rt_b200.config import RopeConfig, rope_inv_freq
    from ds41rt_b200.ops import gemm as G, lib
    k = lib.kernels()
    torch.manual_seed(7)
    rows, IH, ID, ratio, page_rows, max_pages, max_keys = 200, 32, 128, 2, 32, 80, 2560
    pos0 = 3000
    positions = torch.arange(pos0, pos0 + rows, dtype=torch.int32, device="cuda")
    slots = torch.zeros(rows, dtype=torch.int32, device="cuda")
    ldq = IH * ID + 64
    q = torch.randn(rows, ldq, device="cuda").bfloat16()
    w_stride, w_off = 40, 8
    w = torch.randn(rows, w_stride, device="cuda")
    pool = torch.randn(max_pages * page_rows, ID, device="cuda").bfloat16()
    page_table = torch.randperm(max_pages, device="cuda").int().view(1, max_pages).contiguous()
    inv = torch.tensor(rope_inv_freq(RopeConfig(), ID // 2), device="cuda")
    ref = torch.full((rows, max_keys), float("nan"), device="cuda")
    lib.check(k.ds41_index_score(lib.ptr(q), C.c_longlong(ldq), 64, lib.ptr(w), w_stride, w_off, lib.ptr(pool),
                                 lib.ptr(page_table), max_pages, page_rows, lib.ptr(positions), lib.ptr(slots),
                                 lib.ptr(inv), rows, IH, ID, ratio, lib.ptr(ref), max_keys, lib.stream()), "score")
    n_keys = (pos0 + rows) // ratio
    qr = torch.zeros(rows * IH, ID, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(max_keys, ID, device="cuda", dtype=torch.bfloat16)
    vis = torch.zeros(rows, dtype=torch.int32, device="cuda")
    got = torch.full((rows, max_keys), float("nan"), device="cuda")
    st = lib.new_status("cuda")
    lib.check(k.ds41_index_prepare(lib.ptr(q), C.c_longlong(ldq), 64, lib.ptr(pool), lib.ptr(page_table), max_pages,
                                   page_rows, lib.ptr(positions), lib.ptr(slots), lib.ptr(inv), rows, IH, ID, ratio,
                                   n_keys, max_keys, lib.ptr(qr), lib.ptr(kc), lib.ptr(vis), 0, lib.stream()), "prepare")
    G.gemm_raw(qr, kc, got, rows * IH, n_keys, ID, lda=ID, ldb=ID, ldo=max_keys, out_mode=8, bn=256,
               row_w=w[:, w_off:], row_w_ld=w_stride, col_limit=vis, status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "index gemm")
    for r in (0, 57, rows - 1):
        nv = (pos0 + r + 1) // ratio
        assert int(vis[r]) == nv
        a, b = got[r, :nv], ref[r, :nv]
        assert float((a - b).abs().max()) < 2e-3 * float(b.abs().max())
        assert torch.isinf(got[r, nv:n_keys]).all()


def test_fp4_index_keys_and_queries_follow_the_quantisation_oracle():
    """Index keys stored as FP4 rows (E2M1 pairs + UE8M0 per 32 values, 68 bytes for 128 values): the per-key kernel and
    the tensor-core path both score the dequantised keys against queries quantised the same way; the per-key kernel
    also rounds to bf16 where the reference does (dot, weighted relu, head sum)."""
    from ds41rt_b200.config import RopeConfig, rope_inv_freq
    from ds41rt_b200.models.reference import apply_rope
    from ds41rt_b200.ops import gemm as G, lib, quant_ref as Q
    k = lib.kernels()
    torch.manual_seed(9)
    rows, IH, ID, ratio, page_rows, max_pages, max_keys = 70, 32, 128, 2, 32, 40, 1280
    pos0 = 2000
    positions = torch.arange(pos0, pos0 + rows, dtype=torch.int32, device="cuda")
    slots = torch.zeros(rows, dtype=torch.int32, device="cuda")
    ldq = IH * ID
    q = torch.randn(rows, ldq, device="cuda").bfloat16()
    w = torch.rand(rows, IH, device="cuda")
    keys = (torch.randn(max_pages * page_rows, ID, device="cuda") * torch.exp(torch.randn(max_pages * page_rows, 1,
                                                                                             device="cuda"))).bfloat16()
    packed, e = Q.quant_mxfp4(keys.float().cpu(), 32)
    row_bytes = 68
    pool = torch.zeros(max_pages * page_rows, row_bytes, dtype=torch.uint8)
    pool[:, :ID // 2] = packed.view(torch.uint8)
    pool[:, ID // 2:ID // 2 + ID // 32] = e.to(torch.uint8)
    pool = pool.cuda()
    keys_dq = Q.dequant_mxfp4(packed, e, 32).cuda()
    page_table = torch.randperm(max_pages, device="cuda").int().view(1, max_pages).contiguous()
    inv = torch.tensor(rope_inv_freq(RopeConfig(), ID // 2), device="cuda")
    got = torch.full((rows, max_keys), float("nan"), device="cuda")
    lib.check(k.ds41_index_score_cand(lib.ptr(q), C.c_longlong(ldq), 0, lib.ptr(w), IH, 0, lib.ptr(pool),
                                      lib.ptr(page_table), max_pages, page_rows, lib.ptr(positions), lib.ptr(slots),
                                      lib.ptr(inv), rows, IH, ID, ratio, lib.ptr(got), max_keys, None, 0, 0, row_bytes,
                                      lib.stream()), "score")
    n_keys = (pos0 + rows) // ratio
    qr = torch.zeros(rows * IH, ID, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(max_keys, ID, device="cuda", dtype=torch.bfloat16)
    vis = torch.zeros(rows, dtype=torch.int32, device="cuda")
    gemm = torch.full((rows, max_keys), float("nan"), device="cuda")
    st = lib.new_status("cuda")
    lib.check(k.ds41_index_prepare(lib.ptr(q), C.c_longlong(ldq), 0, lib.ptr(pool), lib.ptr(page_table), max_pages,
                                   page_rows, lib.ptr(positions), lib.ptr(slots), lib.ptr(inv), rows, IH, ID, ratio,
                                   n_keys, max_keys, lib.ptr(qr), lib.ptr(kc), lib.ptr(vis), row_bytes, lib.stream()),
              "prepare")
    G.gemm_raw(qr, kc, gemm, rows * IH, n_keys, ID, lda=ID, ldb=ID, ldo=max_keys, out_mode=8, bn=256, row_w=w,
               row_w_ld=IH, col_limit=vis, status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "index gemm")
    # oracle: RoPE, bf16, FP4 round trip of the queries; keys as dequantised; logical key c lives in page_table[c / page_rows]
    qh = q.float().view(rows, IH, ID).cpu()
    qh = apply_rope(qh, positions.cpu().long(), inv.cpu(), ID // 2).bfloat16().float()
    qh = Q.qdq_mxfp4(qh, 32).cuda()
    logical = torch.arange(n_keys, device="cuda")
    phys = page_table[0, logical // page_rows].long() * page_rows + logical % page_rows
    kd = keys_dq[phys]
    assert torch.equal(kc[:n_keys].float(), kd)                                  # gathered keys are the dequantised rows
    # the queries are FP4 values (a fixed point of the round trip) and the round trip of the oracle's RoPE'd queries, up to
    # the few elements where the kernel's and torch's sine differ by an ulp of bf16 before quantisation
    qk = qr.float().view(rows, IH, ID)
    assert torch.equal(Q.qdq_mxfp4(qk.cpu(), 32).cuda(), qk)
    assert float((qk == qh).float().mean()) > 0.97 and float((qk - qh).abs().max()) <= 0.5 * float(qh.abs().max())
    qh = qk
    bf = lambda t: t.bfloat16().float()
    dots = bf(torch.einsum("rhd,cd->rhc", qh, kd))
    want = bf((bf(torch.relu(dots) * w[:, :, None])).sum(1))
    for r in (0, 33, rows - 1):
        nv = (pos0 + r + 1) // ratio
        a, b = got[r, :nv], want[r, :nv]
        assert float((a - b).abs().max()) <= 0.02 * float(b.abs().max())        # bf16 rounding points: one ulp apart at most
        g = gemm[r, :nv]
        assert float((g - b).abs().max()) < 0.02 * float(b.abs().max())
        assert torch.isinf(gemm[r, nv:n_keys]).all()


def test_nvfp4_activation_quantiser_matches_oracle():
    from ds41rt_b200.ops import lib, quant_ref as Q
    from ds41rt_b200.ops.mx import pack_sf_atoms
    k = lib.kernels()
    torch.manual_seed(5)
    rows, K = 70, 768
    x = (torch.randn(rows, K, device="cuda") * torch.exp(torch.randn(rows, 1, device="cuda"))).bfloat16()
    gs = float(x.float().abs().amax() / (448 * 6))
    want_q, want_s, _ = Q.quant_nvfp4(x.float(), gs)
    q = torch.zeros(rows, K // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros((rows + 127) // 128, K // 64, 512, dtype=torch.uint8, device="cuda")
    lib.check(k.ds41_act_quant_nvfp4_rows(lib.ptr(x), C.c_longlong(K), lib.ptr(q), C.c_longlong(K), lib.ptr(sf), rows,
                                          K, C.c_float(gs), None, 1, C.c_longlong(0), C.c_longlong(0), C.c_longlong(0), None,
                                          lib.stream()), "quant")
    torch.cuda.synchronize()
    assert torch.equal(q, want_q)
    want_atoms = pack_sf_atoms(want_s.view(torch.uint8))
    from ds41rt_b200.ops.mx import unpack_sf_atoms
    assert torch.equal(unpack_sf_atoms(sf.cpu(), rows), unpack_sf_atoms(want_atoms.cpu(), rows))


def test_candidate_blocks_select_and_restrict():
    """Candidate layer: block maxima, newest block pinned, best blocks kept (ties to the lowest block id) -> list + mask;
    the masked top-k then only sees keys of those blocks."""
    from ds41rt_b200.ops import lib
    k = lib.kernels()
    rows, max_keys, B, KB, topk = 5, 3000, 8, 40, 64
    torch.manual_seed(1)
    scores = torch.randn(rows, max_keys, device="cuda")
    scores[1] = scores[1].round()                                  # ties between block maxima
    pos = torch.tensor([2999, 2500, 100, 1203, 9], dtype=torch.int32, device="cuda")   # row 2: fewer blocks than KB
    slot = torch.tensor([0, 0, 0, 0, -1], dtype=torch.int32, device="cuda")
    nb = (max_keys + B - 1) // B
    words = (nb + 31) // 32
    blocks = torch.zeros(rows, KB, dtype=torch.int32, device="cuda")
    n_blocks = torch.zeros(rows, dtype=torch.int32, device="cuda")
    mask = torch.full((rows, words), -1, dtype=torch.int32, device="cuda")
    lib.check(k.ds41_candidate_select(lib.ptr(scores), max_keys, lib.ptr(pos), lib.ptr(slot), 1, B, KB, lib.ptr(blocks),
                                      lib.ptr(n_blocks), lib.ptr(mask), words, rows, lib.stream()), "candidate_select")
    sel = torch.zeros(rows, topk, dtype=torch.int32, device="cuda")
    n_sel = torch.zeros(rows, dtype=torch.int32, device="cuda")
    scores2 = torch.randn(rows, max_keys, device="cuda")           # a later layer's scores
    lib.check(k.ds41_topk_select_cand(lib.ptr(scores2), max_keys, lib.ptr(pos), lib.ptr(slot), 1, topk, lib.ptr(sel),
                                      lib.ptr(n_sel), rows, lib.ptr(mask), words, B, lib.stream()), "topk_cand")
    torch.cuda.synchronize()
    bits = mask.cpu().numpy().view("uint32")
    for r in range(4):
        n = int(pos[r]) + 1
        nbv = (n + B - 1) // B
        s = scores[r, :n].cpu()
        s = torch.nn.functional.pad(s, (0, nbv * B - n), value=float("-inf")).view(nbv, B).amax(-1)
        s[(n - 1) // B] = float("inf")
        want = sorted(torch.sort(s, descending=True, stable=True).indices[:KB].tolist())
        got = blocks[r, : int(n_blocks[r])].tolist()
        assert got == want, r
        on = [b for b in range(nb) if (int(bits[r, b >> 5]) >> (b & 31)) & 1]
        assert on == want
        # restricted selection of the later layer
        allowed = torch.zeros(n, dtype=torch.bool)
        for b in want:
            allowed[b * B: (b + 1) * B] = True
        s2 = scores2[r, :n].cpu().masked_fill(~allowed, float("-inf"))
        n_ok = int(allowed.sum())
        order = torch.sort(s2, descending=True, stable=True).indices[: min(topk, n_ok)]
        assert sel[r, : int(n_sel[r])].tolist() == sorted(order.tolist()), r
        assert int(n_sel[r]) == min(topk, n_ok)
    assert int(n_blocks[4]) == 0 and int(n_sel[4]) == 0 and not bits[4].any()


@pytest.mark.parametrize("rows,H", [(300, 512), (1024, 1024)])
def test_hc_mixes_on_the_tensor_cores_match_the_dot_product_kernel(rows, H):
    """Long-pass form of the hyper-connection step: expand without the mixing matrix, the 24 projections from a
    tcgen05 GEMM over the stored streams with the matrix as bf16 high + low parts, hc_finish reading the split-K
    planes.  Streams are identical to the dot-product kernel's; pre / post / comb and the normalised rows agree to
    fp32 rounding of a 4H-long sum, and with the fp32 oracle as closely as the dot-product kernel does."""
    from ds41rt_b200.models import reference as R
    from ds41rt_b200.ops import gemm as G
    from ds41rt_b200.ops import lib
    k = lib.kernels()
    torch.manual_seed(rows)
    K = 4 * H
    streams = torch.randn(rows, 4, H, device="cuda").bfloat16()
    sub = torch.randn(2, rows, H, device="cuda")
    fn = torch.randn(24, K, device="cuda") * 0.5
    scale = torch.tensor([1.0, 0.7, 1.3], device="cuda")
    base = torch.randn(24, device="cuda") * 0.5
    pre_in = torch.rand(rows, 4, device="cuda")
    norm_w = torch.rand(H, device="cuda") + 0.5
    post = torch.rand(rows, 4, device="cuda") * 2
    comb = torch.rand(rows, 16, device="cuda") / 4
    st = lib.new_status("cuda")
    bases = (C.c_void_p * 1)(sub.data_ptr())

    def run(tc, fused=False):
        s = streams.clone()
        partial = torch.zeros(H // 128, rows, 25, device="cuda")
        outs = [torch.zeros(rows, 4, device="cuda"), torch.zeros(rows, 4, device="cuda"),
                torch.zeros(rows, 16, device="cuda"), torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)]
        tap = torch.zeros(rows, H, device="cuda")
        collapse = (lib.ptr(pre_in), lib.ptr(norm_w), lib.ptr(outs[3]), lib.ptr(tap), C.c_float(1e-20)) if fused else \
            (lib.ptr(None), lib.ptr(None), lib.ptr(None), lib.ptr(None), C.c_float(0.0))
        lib.check(k.ds41_hc_post_mix(lib.ptr(s), lib.ptr(s), bases, 1, 2, C.c_longlong(rows * H), lib.ptr(post),
                                     lib.ptr(comb), lib.ptr(None if tc else fn), lib.ptr(partial), rows, H,
                                     lib.ptr(None), lib.ptr(None), lib.ptr(st), *collapse, lib.stream()), "post_mix")
        mix = (lib.ptr(None), 0, C.c_longlong(0), 0)
        keep = None
        if tc:
            hi = fn.bfloat16()
            w = torch.zeros(64, K, device="cuda", dtype=torch.bfloat16)
            w[:24], w[24:48] = hi, (fn - hi.float()).bfloat16()
            splits = G.pick_splits(rows, K, max_splits=16)
            assert splits > 1
            planes = torch.zeros(splits, rows, 64, device="cuda")
            G.gemm_raw(s.view(rows, K), w, None, rows, 64, K, lda=K, ldb=K, ldo=64, out_mode=1, k_splits=splits,
                       split_workspace=planes, bn=64, status=st, static_operand=2)
            mix = (lib.ptr(planes), splits, C.c_longlong(rows * 64), 64)
            keep = (w, planes)
        lib.check(k.ds41_hc_finish(lib.ptr(partial), 1 if tc else H // 128, lib.ptr(scale), lib.ptr(base), lib.ptr(pre_in),
                                   lib.ptr(s), lib.ptr(norm_w), lib.ptr(outs[0]), lib.ptr(outs[1]), lib.ptr(outs[2]),
                                   lib.ptr(None if fused else outs[3]), lib.ptr(None if fused else tap), lib.ptr(None),
                                   lib.ptr(None), rows, H, 20, C.c_float(1e-6), C.c_float(1e-20), *mix, lib.stream()),
                  "finish")
        torch.cuda.synchronize()
        lib.raise_on_status(st, "hc mixes")
        return s, outs + [tap], partial, keep

    s_a, a, part_a, _ = run(False)
    s_b, b, part_b, _ = run(True)
    s_c, c, part_c, _ = run(True, fused=True)       # expand kernel also collapses and normalises; finish: mixes only
    assert torch.equal(s_a, s_b) and torch.equal(s_b, s_c)
    assert torch.equal(b[3], c[3]) and torch.equal(b[4], c[4]) and torch.equal(part_b[0, :, 24], part_c[0, :, 24])
    for x, y in zip(b[:3], c[:3]):
        assert float((x - y).abs().max()) < 1e-5          # the split-K planes are summed in another order
    assert torch.allclose(part_a[:, :, 24].sum(0), part_b[0, :, 24], rtol=1e-5, atol=1e-4)   # sums of squares
    assert torch.equal(a[3], b[3])                                                       # collapse + norm: same inputs
    for x, y in zip(a[:3], b[:3]):
        assert float((x - y).abs().max()) < 2e-4
    pre1, post1, comb1 = R.hc_mixes(s_b.float().cpu(), fn.cpu(), scale.cpu(), base.cpu(), 4, 20, 1e-6, 1e-20)
    assert float((b[0].cpu() - pre1).abs().max()) < 1e-3
    assert float((b[1].cpu() - post1).abs().max()) < 1e-3
    assert float((b[2].cpu().view(rows, 4, 4) - comb1).abs().max()) < 1e-3
