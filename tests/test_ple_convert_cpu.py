"""Engram table conversion FP8 -> NVFP4 on the CPU: native code against an independent fp32 statement of the recipe,
streaming with resume, and refusal of NaN tables."""
import json
import os

import numpy as np
import pytest
import torch

from ds41rt_b200.models.engram import dequant_rows_reference, random_table_rows
from ds41rt_b200.runtime import ple_convert as P


def _recipe(rows_q: torch.Tensor, dim: int):
    """(records uint8 [n, dim/2 + dim/16], table scale) by plain fp32 torch arithmetic."""
    n = rows_q.shape[0]
    vals = dequant_rows_reference(rows_q, dim)                       # fp32, exact
    amax = vals.abs().max()
    scale = amax / torch.tensor(6.0 * 448.0)
    g = vals.abs().view(n, dim // 16, 16)
    top = g.amax(-1)
    want = (top / (torch.tensor(6.0) * scale)).clamp(2.0 ** -9, 448.0)
    want = torch.where(top > 0, want, torch.ones_like(want))
    sc8 = want.to(torch.float8_e4m3fn)
    q = g / (sc8.float() * scale)[..., None]
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    mids = (grid[1:] + grid[:-1]) / 2
    code = torch.zeros_like(q, dtype=torch.int64)
    for i, m in enumerate(mids):                                     # a tie moves on only from an odd code
        code = torch.where((q > m) | ((q == m) & (i % 2 == 1)), torch.full_like(code, i + 1), code)
    src = rows_q[:, :dim].to(torch.int64).view(n, dim // 16, 16)
    code = code | (((src & 128) != 0) & ((src & 127) != 0)).to(torch.int64) * 8
    code = code.view(n, dim // 2, 2)
    payload = (code[..., 0] | (code[..., 1] << 4)).to(torch.uint8)
    return torch.cat([payload, sc8.view(torch.uint8)], dim=1), float(scale)


@pytest.mark.parametrize("dim", [256, 64])
def test_native_conversion_equals_the_fp32_recipe_bit_for_bit(dim):
    rows = random_table_rows(513, row_dim=dim, row_bytes=dim + dim // 32, seed=3)
    rows[7, :16] = 0                                                # an all-zero group: scale 1.0, +0 codes
    rows[9, 0] = 0x80                                               # a negative zero stays +0
    rows[11, dim:dim + dim // 32] = 90                              # a tiny group far below the table scale
    src = rows.numpy()
    amax = P.scan_rows(src, dim, threads=3)
    want, want_scale = _recipe(rows, dim)
    assert amax == float(dequant_rows_reference(rows, dim).abs().max())
    scale = P.global_scale(amax)
    assert scale == want_scale
    got = torch.from_numpy(P.convert_rows(src, scale, dim, threads=3))
    assert torch.equal(got[:, dim // 2:], want[:, dim // 2:])        # block scales
    assert torch.equal(got[:, :dim // 2], want[:, :dim // 2])        # codes
    assert got[7, dim // 2] == 0x38 and int(got[7, :8].sum()) == 0 and (got[9, 0] & 15) != 8
    # reconstruction: every value within half a code step of its group (scale rounding included)
    back = P.dequant_rows_reference(got, scale, dim)
    ref = dequant_rows_reference(rows, dim)
    step = got[:, dim // 2:].view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=1) * scale
    assert bool(((back - ref).abs() <= 1.0 * step + 1e-12).all())
    rel = float((back - ref).norm() / ref.norm())
    assert rel < 0.12, rel


def test_a_nan_payload_or_scale_is_refused():
    rows = random_table_rows(64, seed=1)
    rows[5, 3] = 0x7F
    assert np.isnan(P.scan_rows(rows.numpy()))
    rows = random_table_rows(64, seed=1)
    rows[6, 256 + 2] = 255
    assert np.isnan(P.scan_rows(rows.numpy()))


def test_streamed_conversion_resumes_and_matches_one_shot(tmp_path):
    n, dim = 1000, 256
    rows = random_table_rows(n, seed=5)
    src, dst = str(tmp_path / "t.bin"), str(tmp_path / "t.nvfp4.bin")
    rows.numpy().tofile(src)
    part = P.convert_table(src, dst, n, dim, threads=2, chunk_rows=128, stop_after_chunks=3)
    assert part["complete"] is False and part["scanned_chunks"] == 3
    part = P.convert_table(src, dst, n, dim, threads=2, chunk_rows=128, stop_after_chunks=8)      # 5 scans + 3 records chunks
    assert part["complete"] is False and part["amax"] is not None and 0 < part["converted_chunks"] < 8
    mark = part["converted_chunks"]
    meta = P.convert_table(src, dst, n, dim, threads=2, chunk_rows=128)
    assert meta["complete"] and meta["row_bytes"] == 144 and meta["format"] == "nvfp4"
    with open(dst + ".progress.json") as f:
        assert json.load(f)["converted_chunks"] == 8 and mark < 8
    one_shot = P.convert_rows(rows.numpy(), meta["global_scale"], dim)
    assert np.array_equal(np.fromfile(dst, dtype=np.uint8).reshape(n, 144), one_shot)
    with open(dst + ".json") as f:
        assert json.load(f)["global_scale"] == meta["global_scale"]
    # a changed source invalidates the progress record
    rows[0, 0] ^= 1
    rows.numpy().tofile(src)
    again = P.convert_table(src, dst, n, dim, threads=2, chunk_rows=128, stop_after_chunks=1)
    assert again["scanned_chunks"] == 1 and again["converted_chunks"] == 0


def test_wrong_file_size_is_an_error(tmp_path):
    src = str(tmp_path / "t.bin")
    random_table_rows(10, seed=0).numpy().tofile(src)
    with pytest.raises(ValueError):
        P.convert_table(src, str(tmp_path / "o.bin"), 11)
