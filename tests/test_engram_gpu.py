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


@pytest.mark.parametrize("rows", [5, 40])
def test_engine_pass_with_engram_layer_matches_oracle(rows):
    """A decoder layer that has an Engram memory: the engine's split hyper-connection step (expand, gated update,
    mixes recomputed, collapse) against the fp32 oracle with the same update on entry to that layer."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.engram import (EngramLayer, dequant_rows_reference, engram_reference,
                                            init_engram_weights, random_table_rows)
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.weights import init_weights
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=3)
    dev = torch.device("cuda", 0)
    H, rpt, dim = cfg.hidden, 24, 256
    wkv, q_w, k_w = init_engram_weights(H, seed=5, std=0.002)
    bf = lambda t: t.bfloat16()
    table = random_table_rows(rows * rpt, seed=7)
    mask = torch.ones(rows, dtype=torch.uint8)
    mask[2] = 0
    tokens = torch.randint(0, cfg.vocab - 8, (rows,), generator=torch.Generator().manual_seed(rows))

    ref = ReferenceModel(cfg, w)
    deq = dequant_rows_reference(table, dim).bfloat16().view(rows, rpt * dim)
    ref.engram_hook = lambda l, s: engram_reference(s.bfloat16(), deq, bf(wkv), bf(q_w), bf(k_w), mask) if l == 1 else s
    want = ref.forward(tokens)
    plain = ReferenceModel(cfg, w).forward(tokens)
    assert float((want - plain).abs().max()) > 1e-2            # the update matters in this setup

    eng = DS41Engine(cfg, EngineWeights.from_fp32(cfg, w, 0, 1, dev), max_rows=max(rows, 8), slots=1, max_ctx=256)
    eng.attach_engram(1, EngramLayer(bf(wkv).to(dev), bf(q_w).to(dev), bf(k_w).to(dev), H))
    assert eng.cache.ensure(0, rows)
    eng.set_rows(tokens.tolist(), list(range(rows)), [0] * rows)
    eng.set_engram_rows(1, table.numpy(), mask)
    eng.forward_rows(rows)
    torch.cuda.synchronize()
    eng.check_status("engram pass")
    got = eng.logits_rows(rows).float().cpu()
    # bf16 activations may flip near-tied expert / key selections in single rows, so judge the bulk of the rows
    scale = float(want.abs().max())
    err = (got - want).abs().max(dim=1).values
    off = (got - plain).abs().max(dim=1).values
    assert float(err.median()) < 0.05 * scale, (float(err.median()), scale)
    assert int((err < off).sum()) >= 0.8 * rows, (err, off)
    # and without rows for this pass the layer is skipped
    eng.clear_engram_rows()
    eng.cache.release(0)
    assert eng.cache.ensure(0, rows)
    eng.set_rows(tokens.tolist(), list(range(rows)), [0] * rows)
    eng.forward_rows(rows)
    torch.cuda.synchronize()
    got2 = eng.logits_rows(rows).float().cpu()
    assert float((got2 - plain).abs().max(dim=1).values.median()) < 0.05 * float(plain.abs().max())


def test_nvfp4_table_rows_dequantise_exactly_and_drive_the_layer():
    """A table converted on the CPU (FP8 -> NVFP4) read back by the GPU: bf16((code * scale) * table scale) bit for bit,
    and the layer's update from those rows against the fp32 reference."""
    from ds41rt_b200.models.engram import EngramLayer, engram_reference, random_table_rows
    from ds41rt_b200.ops import lib
    from ds41rt_b200.runtime import ple_convert as P
    dev = torch.device("cuda")
    T, H, rpt, dim = 12, 512, 24, 256
    src = random_table_rows(T * rpt, seed=4)
    scale = P.global_scale(P.scan_rows(src.numpy()))
    rows_q = torch.from_numpy(P.convert_rows(src.numpy(), scale))
    assert rows_q.shape == (T * rpt, 144)
    g = torch.Generator(device=dev).manual_seed(1)
    wkv = (torch.randn(5 * H, rpt * dim, device=dev, generator=g) * 0.02).bfloat16()
    q_w = (torch.randn(4, H, device=dev, generator=g) * 0.5 + 1).bfloat16()
    k_w = (torch.randn(4, H, device=dev, generator=g) * 0.5 + 1).bfloat16()
    x = torch.randn(T, 4, H, device=dev, generator=g).bfloat16()
    layer = EngramLayer(wkv, q_w, k_w, H, max_tokens=16, table_format="nvfp4", table_scale=scale)
    assert layer.row_bytes == 144
    got = layer.forward(x.clone(), rows_q.numpy(), None)
    torch.cuda.synchronize()
    lib.raise_on_status(layer.status, "engram wkv")
    deq = P.dequant_rows_reference(rows_q, scale, dim).bfloat16()
    assert torch.equal(layer.rows[:T].cpu().view(-1, dim), deq)
    want = engram_reference(x.cpu(), deq.view(T, rpt * dim), wkv.cpu(), q_w.cpu(), k_w.cpu(), None)
    err = float((got.float().cpu() - want).abs().max())
    assert err < 3e-2 * float(want.abs().max()), err
    k = lib.kernels()
    assert k.ds41_engram_dequant_nvfp4(lib.ptr(layer.staging), 144, dim, __import__("ctypes").c_float(0.0),
                                       lib.ptr(layer.rows), 4, lib.stream()) != 0          # a zero table scale is refused


@pytest.mark.parametrize("rows,H", [(1, 5120), (37, 5120), (300, 2048)])
def test_wire_records_round_trip(rows, H):
    """Hidden-state rows as E4M3 + UE8M0/32 records: the encoder equals its fp32 statement byte for byte, the decoder
    equals the reference decode rule, and the round trip stays within E4M3's half-step of each group's scale."""
    from ds41rt_b200.ops import wire as W
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(rows)
    x = (torch.randn(rows, H, device=dev, generator=g) * torch.rand(rows, 1, device=dev, generator=g) * 8).bfloat16()
    x[0, :32] = 0                                                 # an all-zero group
    x[0, 32] = 448.0                                              # an exact power-of-two ratio
    rec = W.encode(x)
    assert rec.shape == (rows, W.record_bytes(H)) and (H != 5120 or rec.shape[1] == 5280)
    want = W.encode_reference(x)
    n = H + H // 32
    assert torch.equal(rec[:, :n], want[:, :n])
    y = W.decode(rec, H)
    assert torch.equal(y, W.decode_reference(rec, H))
    scale = torch.pow(2.0, rec[:, H:n].float() - 127).repeat_interleave(32, dim=1)
    assert bool(((y.float() - x.float()).abs() <= scale * 16 + 1e-30).all())     # half of E4M3's largest step (32)
    rel = float((y.float() - x.float()).norm() / x.float().norm())
    assert rel < 0.04, rel
    # strided bf16 views and a NaN scale byte
    wide = torch.zeros(rows, H + 64, dtype=torch.bfloat16, device=dev)
    W.decode(rec, H, out=wide[:, :H])
    assert torch.equal(wide[:, :H], y) and float(wide[:, H:].abs().sum()) == 0.0
    rec[0, H] = 255
    assert bool(torch.isnan(W.decode(rec, H)[0, :32]).all())
