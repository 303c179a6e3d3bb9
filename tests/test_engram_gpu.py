"""Engram GPU path (row dequant, wkv projection on the tcgen05 GEMM, gated stream update) vs the PyTorch reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H", [(5, 512), (40, 5120)])
def test_engram_layer_matches_reference(T, H):
    from ds41rt_b200.models.engram import EngramLayer, dequant_rows_reference, engram_reference
    from ds41rt_b200.ops import lib
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(T)
    rpt, dim, rb = 24, 256, 264
    rows_q = torch.zeros(T * rpt, rb, dtype=torch.uint8, device=dev)
    payload = (torch.randn(T * rpt, dim, device=dev, generator=g) * 2).to(torch.float8_e4m3fn)
    rows_q[:, :dim] = payload.view(torch.uint8)
    rows_q[:, dim:] = torch.randint(120, 130, (T * rpt, 8), device=dev, generator=g, dtype=torch.uint8)
    rows_q[0, dim] = 0                                            # the 2^-127 scale
    wkv = (torch.randn(5 * H, rpt * dim, device=dev, generator=g) * 0.02).bfloat16()
    q_w = (torch.randn(4, H, device=dev, generator=g) * 0.5 + 1).bfloat16()
    k_w = (torch.randn(4, H, device=dev, generator=g) * 0.5 + 1).bfloat16()
    x = torch.randn(T, 4, H, device=dev, generator=g).bfloat16()
    mask = torch.ones(T, dtype=torch.uint8, device=dev)
    mask[1] = 0                                                   # an image position passes through
    layer = EngramLayer(wkv, q_w, k_w, H, max_tokens=64)
    deq = dequant_rows_reference(rows_q.cpu(), dim).bfloat16()
    want = engram_reference(x.cpu(), deq.view(T, rpt * dim), wkv.cpu(), q_w.cpu(), k_w.cpu(), mask.cpu())
    got = layer.forward(x.clone(), rows_q.cpu().numpy(), mask)
    torch.cuda.synchronize()
    lib.raise_on_status(layer.status, "engram wkv")
    assert torch.equal(layer.rows[:T].cpu().view(-1, dim), deq)   # dequantisation is exact
    err = float((got.float().cpu() - want).abs().max())
    assert err < 3e-2 * float(want.abs().max()), err
    assert torch.equal(got[1].cpu(), x[1].cpu())
