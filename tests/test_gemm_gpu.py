"""tcgen05 GEMM kernel vs a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


def _rel(out, ref):
    return float((out.float() - ref).abs().max() / ref.abs().max().clamp(min=1e-6))


@pytest.mark.parametrize("rows,N,K", [(1, 256, 512), (5, 1280, 5120), (16, 384, 1024), (64, 512, 192),
                                      (100, 640, 2304), (300, 1024, 512), (1000, 768, 1536), (300, 200, 512),
                                      (257, 72, 256)])
def test_matmul_nt_bf16(rows, N, K):
    from ds41rt_b200.ops import gemm as G, lib
    torch.manual_seed(rows + N)
    x = torch.randn(rows, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    st = lib.new_status("cuda")
    out = G.matmul_nt(x, w, status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm")
    assert _rel(out, _ref(x, w)) < 1e-2
    out32 = G.matmul_nt(x, w, out_dtype=torch.float32, status=st)
    torch.cuda.synchronize()
    assert _rel(out32, _ref(x, w)) < 2e-3


@pytest.mark.parametrize("rows,N,K,splits", [(4, 1792, 5120, 8), (8, 512, 1024, 4), (33, 384, 512, 2)])
def test_split_k_planes(rows, N, K, splits):
    from ds41rt_b200.ops import gemm as G, lib
    x = torch.randn(rows, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    planes = torch.zeros(splits, rows, N, device="cuda")
    st = lib.new_status("cuda")
    G.linear_planes(x, w, planes, splits, status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm split")
    assert _rel(planes.sum(0), _ref(x, w)) < 2e-3


def test_batched_grouped_output():
    """wo_a shape: per-group weights [G, o, k], activations [rows, G*k] -> [rows, G*o]."""
    from ds41rt_b200.ops import gemm as G, lib
    g, o, k, rows = 2, 256, 1024, 6
    w = (torch.randn(g, o, k, device="cuda") * 0.05).bfloat16()
    x = torch.randn(rows, g * k, device="cuda").bfloat16()
    out = torch.zeros(rows, g * o, device="cuda", dtype=torch.bfloat16)
    st = lib.new_status("cuda")
    G.gemm_raw(w, x, out, o, rows, k, lda=k, ldb=g * k, ldo=g * o, out_mode=2, batch=g, a_batch_stride=o * k,
               b_batch_stride=k, out_batch_stride=o, status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm batched")
    ref = torch.einsum("rgk,gok->rgo", x.float().view(rows, g, k), w.float()).reshape(rows, g * o)
    assert _rel(out, ref) < 1e-2


def test_fp8_unscaled():
    from ds41rt_b200.ops import gemm as G, lib
    rows, N, K = 7, 512, 1024
    x = torch.randn(rows, K, device="cuda").to(torch.float8_e4m3fn)
    w = torch.randn(N, K, device="cuda").to(torch.float8_e4m3fn)
    out = torch.zeros(rows, N, device="cuda")
    st = lib.new_status("cuda")
    G.gemm_raw(w, x, out, N, rows, K, lda=K, ldb=K, ldo=N, kind=1, out_mode=3, status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm fp8")
    assert _rel(out, _ref(x, w)) < 1e-3


@pytest.mark.parametrize("rows,N,K", [(5, 256, 512), (40, 384, 1024), (128, 256, 256), (300, 256, 512)])
def test_mxfp8_block_scaled(rows, N, K):
    from ds41rt_b200.ops import gemm as G, lib, quant_ref as Q
    from ds41rt_b200.ops.mx import pack_sf_atoms
    torch.manual_seed(1)
    x = torch.randn(rows, K, device="cuda") * torch.exp(torch.randn(rows, 1, device="cuda"))
    w = torch.randn(N, K, device="cuda") * 0.1 * torch.exp(torch.randn(N, 1, device="cuda"))
    xq, xe = Q.quant_mxfp8(x)
    wq, we = Q.quant_mxfp8(w)
    ref = Q.dequant_mxfp8(xq, xe) @ Q.dequant_mxfp8(wq, we).t()
    st = lib.new_status("cuda")
    out = torch.zeros(rows, N, device="cuda")
    sfx, sfw = pack_sf_atoms(xe), pack_sf_atoms(we)
    if rows <= 128:
        G.gemm_raw(wq, xq, out, N, rows, K, lda=K, ldb=K, ldo=N, kind=2, out_mode=3, sfa=sfw, sfb=sfx,
                   bn=max(32, G.pick_bn(rows)), status=st)
    else:
        G.gemm_raw(xq, wq, out, rows, N, K, lda=K, ldb=K, ldo=N, kind=2, out_mode=1, sfa=sfx, sfb=sfw, bn=128,
                   status=st)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm mx")
    assert _rel(out, ref) < 2e-3


@pytest.mark.parametrize("rows,N,K", [(5, 256, 512), (40, 384, 1024), (16, 4608, 5120)])
def test_mxfp4_weights_times_mxfp8_rows(rows, N, K):
    """E2M1 weights (two per byte, UE8M0 per 32) as the M operand of the block-scaled kind, E4M3 rows as N."""
    from ds41rt_b200.ops import gemm as G, lib, quant_ref as Q
    from ds41rt_b200.ops.mx import pack_sf_atoms
    torch.manual_seed(2)
    x = torch.randn(rows, K, device="cuda") * torch.exp(torch.randn(rows, 1, device="cuda"))
    w = torch.randn(N, K, device="cuda") * 0.1 * torch.exp(torch.randn(N, 1, device="cuda"))
    xq, xe = Q.quant_mxfp8(x)
    wq, we = Q.quant_mxfp4(w)
    ref = Q.dequant_mxfp8(xq, xe) @ Q.dequant_mxfp4(wq, we).t()
    st = lib.new_status("cuda")
    out = torch.zeros(rows, N, device="cuda")
    G.gemm_raw(wq.contiguous(), xq, out, N, rows, K, lda=K, ldb=K, ldo=N, kind=2, out_mode=3, sfa=pack_sf_atoms(we),
               sfb=pack_sf_atoms(xe), bn=max(32, G.pick_bn(rows)), status=st, a_format=1)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm mxfp4")
    assert _rel(out, ref) < 2e-3


@pytest.mark.parametrize("rows,N,K", [(5, 256, 512), (40, 384, 1024), (16, 4608, 5120), (300, 256, 768)])
def test_nvfp4_both_operands(rows, N, K):
    """E2M1 values with an E4M3 scale per 16 elements and one fp32 scale per tensor (NVFP4) on both operands:
    tcgen05 kind::mxf4nvf4, scale_vec 4X, global scales folded into the epilogue."""
    from ds41rt_b200.ops import gemm as G, lib, quant_ref as Q
    from ds41rt_b200.ops.mx import pack_sf_atoms
    torch.manual_seed(3)
    x = torch.randn(rows, K, device="cuda") * torch.exp(0.5 * torch.randn(rows, 1, device="cuda"))
    w = torch.randn(N, K, device="cuda") * 0.1 * torch.exp(0.5 * torch.randn(N, 1, device="cuda"))
    xq, xs, xg = Q.quant_nvfp4(x)
    wq, ws, wg = Q.quant_nvfp4(w)
    ref = Q.dequant_nvfp4(xq, xs, xg) @ Q.dequant_nvfp4(wq, ws, wg).t()
    st = lib.new_status("cuda")
    out = torch.zeros(rows, N, device="cuda")
    sfx = pack_sf_atoms(xs.view(torch.uint8))
    sfw = pack_sf_atoms(ws.view(torch.uint8))
    alpha = float(xg) * float(wg)
    if rows <= 128:
        G.gemm_raw(wq.contiguous(), xq.contiguous(), out, N, rows, K, lda=K, ldb=K, ldo=N, kind=3, out_mode=3, sfa=sfw,
                   sfb=sfx, bn=max(32, G.pick_bn(rows)), status=st, alpha=alpha)
    else:
        G.gemm_raw(xq.contiguous(), wq.contiguous(), out, rows, N, K, lda=K, ldb=K, ldo=N, kind=3, out_mode=1, sfa=sfx,
                   sfb=sfw, bn=128, status=st, alpha=alpha)
    torch.cuda.synchronize()
    lib.raise_on_status(st, "gemm nvfp4")
    assert _rel(out, ref) < 2e-3
