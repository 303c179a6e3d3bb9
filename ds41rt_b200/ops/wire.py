"""Hidden-state rows as wire records: H E4M3 values followed by H/32 UE8M0 scales (one per 32 values) per row.

`encode` / `decode` run the CUDA kernels of csrc/kernels/wire.cu; `encode_reference` / `decode_reference` are the plain
PyTorch statements of the same arithmetic for the tests.  A record of H = 5120 is 5280 bytes against 10240 for bf16.
Record layout and decode rule: native/cuda/kernels/v41_exl3_wire.cu:9-18 of the reference.
"""
from __future__ import annotations

import torch

from . import lib


def record_bytes(H: int) -> int:
    assert H % 32 == 0
    return (H + H // 32 + 7) // 8 * 8


def encode(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [rows, H] (last dimension contiguous) -> uint8 [rows, record_bytes(H)] on the current stream."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    rows, H = x.shape
    rb = record_bytes(H)
    if out is None:
        out = torch.empty(rows, rb, dtype=torch.uint8, device=x.device)
    assert out.shape == (rows, rb) and out.dtype == torch.uint8 and out.is_contiguous()
    lib.check(lib.kernels().ds41_wire_encode(lib.ptr(x), x.stride(0), lib.ptr(out), rb, rows, H, lib.stream()),
              "wire_encode")
    return out


def decode(records: torch.Tensor, H: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """uint8 [rows, record_bytes(H)] -> bf16 [rows, H] on the current stream."""
    assert records.is_cuda and records.dtype == torch.uint8 and records.dim() == 2 and records.is_contiguous()
    rows, rb = records.shape
    assert rb == record_bytes(H)
    if out is None:
        out = torch.empty(rows, H, dtype=torch.bfloat16, device=records.device)
    assert out.shape == (rows, H) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    lib.check(lib.kernels().ds41_wire_decode(lib.ptr(records), rb, lib.ptr(out), out.stride(0), rows, H, lib.stream()),
              "wire_decode")
    return out


def encode_reference(x: torch.Tensor) -> torch.Tensor:
    """fp32 statement of the encoder: scale = 2^ceil(log2(max(amax * fl(1/448), 2^-126))) per 32 values (the product in
    fp32, as the kernel forms it), payload = e4m3(x / scale)."""
    rows, H = x.shape
    g = x.float().view(rows, H // 32, 32)
    t = (g.abs().amax(-1) * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=x.device)).clamp(min=2.0 ** -126)
    m, e = torch.frexp(t)                               # t = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e).clamp(max=127)  # exact powers of two keep their exponent
    payload = (g * torch.pow(2.0, -e.float())[..., None]).to(torch.float8_e4m3fn).view(torch.uint8).view(rows, H)
    out = torch.zeros(rows, record_bytes(H), dtype=torch.uint8, device=x.device)
    out[:, :H] = payload
    out[:, H:H + H // 32] = (e + 127).to(torch.uint8)
    return out


def decode_reference(records: torch.Tensor, H: int) -> torch.Tensor:
    """fp32 statement of the decoder, rounded to bf16."""
    vals = records[:, :H].contiguous().view(torch.float8_e4m3fn).float()
    e = records[:, H:H + H // 32].to(torch.int32)
    scale = torch.where(e == 0, torch.tensor(2.0 ** -127, device=records.device), torch.pow(2.0, (e - 127).float()))
    scale = torch.where(e == 255, torch.tensor(float("nan"), device=records.device), scale)
    return (vals * scale.repeat_interleave(32, dim=1)).bfloat16()
