"""Engram memory layer: hashed n-gram rows -> key/value projection -> gated update of the residual streams.

Per token: the (2,3,4)-gram hashes of its history give `n_heads * 3` row ids into the layer's table (csrc/core/engram.cc
computes them, `runtime/engram_io.py` gathers the rows on a host thread).  On the GPU the rows are dequantised
(`ds41_engram_dequant`), multiplied by `engram.wkv` ([(4 + 1) * H, 24 * 256], tcgen05 GEMM) into four keys and one
value per token, and `ds41_engram_gate` adds gate * value to each of the four streams.

`engram_reference` is the plain PyTorch fp32 statement of the same update used by the tests.
Reference: config rust/crates/ds41rt-loader/src/v41_config.rs:131-144, hashing rust/crates/ds41rt-core/src/engram.rs:19-78,
kernels native/cuda/kernels/engram.cu:19-110, pass integration rust/crates/ds41rt-daemon/src/v41_target_pass.rs:403-442.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops import gemm as G
from ..ops import lib


def dequant_rows_reference(rows_q: torch.Tensor, dim: int = 256) -> torch.Tensor:
    """uint8 [n, >= dim + dim/32] -> fp32 [n, dim] (e4m3 payload, UE8M0 scale per 32; exponent 0 = 2^-127)."""
    payload = rows_q[:, :dim].contiguous().view(torch.float8_e4m3fn).float()
    e = rows_q[:, dim:dim + dim // 32].to(torch.int32)
    scale = torch.where(e == 0, torch.tensor(2.0 ** -127), torch.pow(2.0, (e - 127).float()))
    return payload * scale.repeat_interleave(32, dim=1)


def engram_reference(x: torch.Tensor, rows_deq: torch.Tensor, wkv: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor,
                     text_mask: Optional[torch.Tensor] = None, eps: float = 1e-20) -> torch.Tensor:
    """x [T, 4, H], rows_deq [T, 24*256] (bf16-rounded), wkv [5H, 24*256] -> updated streams [T, 4, H] (fp32 math with the
    kernel's bf16 rounding points: projection output and result)."""
    T, S, H = x.shape
    kv = (rows_deq.float() @ wkv.float().t()).bfloat16().float().view(T, S + 1, H)
    key, val = kv[:, :S], kv[:, S]
    xf = x.float()
    dot = (xf * (q_w.float() * k_w.float())[None] * key).sum(-1)
    dot = dot * torch.rsqrt((xf * xf).mean(-1) + eps) * torch.rsqrt((key * key).mean(-1) + eps) / (H ** 0.5)
    gate = torch.sigmoid(torch.sign(dot) * torch.sqrt(dot.abs().clamp(min=1e-6)))
    out = (xf + gate[..., None] * val[:, None]).bfloat16().float()
    if text_mask is not None:
        out = torch.where(text_mask.bool()[:, None, None], out, xf)
    return out


class EngramLayer:
    def __init__(self, wkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, hidden: int,
                 rows_per_token: int = 24, row_dim: int = 256, row_bytes: int = 264, max_tokens: int = 64,
                 eps: float = 1e-20):
        """wkv [5 * hidden, rows_per_token * row_dim] bf16, q_weight / k_weight [4, hidden] bf16."""
        dev = wkv.device
        assert wkv.shape == (5 * hidden, rows_per_token * row_dim) and wkv.dtype == torch.bfloat16
        self.wkv, self.q_w, self.k_w = wkv.contiguous(), q_weight.contiguous(), k_weight.contiguous()
        self.H, self.rpt, self.dim, self.row_bytes, self.eps = hidden, rows_per_token, row_dim, row_bytes, eps
        self.max_tokens = max_tokens
        self.staging = torch.zeros(max_tokens * rows_per_token, row_bytes, dtype=torch.uint8, device=dev)
        self.rows = torch.zeros(max_tokens, rows_per_token * row_dim, dtype=torch.bfloat16, device=dev)
        self.kv = torch.zeros(max_tokens, 5 * hidden, dtype=torch.bfloat16, device=dev)
        self.status = lib.new_status(dev)

    def forward(self, streams: torch.Tensor, rows_q_host, text_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """streams [T, 4, H] bf16 (updated in place), rows_q_host: uint8 [T * rows_per_token, row_bytes] (numpy or a
        pinned tensor, e.g. a gather slot).  Asynchronous on the current stream after the upload."""
        T = streams.shape[0]
        assert T <= self.max_tokens and streams.dtype == torch.bfloat16 and streams.is_contiguous()
        k, st = lib.kernels(), lib.stream
        src = rows_q_host if isinstance(rows_q_host, torch.Tensor) else torch.from_numpy(rows_q_host)
        n = T * self.rpt
        self.staging[:n].copy_(src[:n], non_blocking=True)
        lib.check(k.ds41_engram_dequant(lib.ptr(self.staging), self.row_bytes, self.dim, lib.ptr(self.rows), n, st()),
                  "engram_dequant")
        G.matmul_nt(self.rows[:T], self.wkv, self.kv[:T], status=self.status)
        lib.check(k.ds41_engram_gate(lib.ptr(streams), lib.ptr(self.kv), lib.ptr(self.q_w), lib.ptr(self.k_w),
                                     lib.ptr(text_mask), lib.ptr(streams), T, self.H, C.c_float(self.eps), st()),
                  "engram_gate")
        return streams
