"""Engram memory layer: hashed n-gram rows -> key/value projection -> gated update of the residual streams.

Per token: the (2,3,4)-gram hashes of its history give `n_heads * 3` row ids into the layer's table (csrc/core/engram.cc
computes them, `runtime/engram_io.py` gathers the rows on a host thread).  On the GPU the rows are dequantised
(`ds41_engram_dequant`; `ds41_engram_dequant_nvfp4` for a table converted by `runtime/ple_convert.py`), multiplied by `engram.wkv` ([(4 + 1) * H, 24 * 256], tcgen05 GEMM) into four keys and one
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
                 rows_per_token: int = 24, row_dim: int = 256, row_bytes: Optional[int] = None, max_tokens: int = 64,
                 eps: float = 1e-20, table_format: str = "fp8", table_scale: float = 1.0):
        """wkv [5 * hidden, rows_per_token * row_dim] bf16, q_weight / k_weight [4, hidden] bf16.
        table_format "fp8": records of row_dim E4M3 values + row_dim/32 UE8M0 scales (264 bytes for 256);
        "nvfp4": records of row_dim/2 E2M1 pair bytes + row_dim/16 E4M3 scales (144 bytes) with the table's fp32
        scale `table_scale` (runtime/ple_convert.py writes both)."""
        dev = wkv.device
        assert wkv.shape == (5 * hidden, rows_per_token * row_dim) and wkv.dtype == torch.bfloat16
        assert table_format in ("fp8", "nvfp4")
        if row_bytes is None:
            row_bytes = row_dim + row_dim // 32 if table_format == "fp8" else row_dim // 2 + row_dim // 16
        self.wkv, self.q_w, self.k_w = wkv.contiguous(), q_weight.contiguous(), k_weight.contiguous()
        self.H, self.rpt, self.dim, self.row_bytes = hidden, rows_per_token, row_dim, row_bytes
        self.table_format, self.table_scale = table_format, float(table_scale)
        self.eps = eps
        self.max_tokens = 0
        self.status = lib.new_status(dev)
        self.reserve(max_tokens)

    def reserve(self, max_tokens: int) -> None:
        """Size the device buffers for passes of up to `max_tokens` rows (no allocation happens in forward)."""
        if max_tokens <= self.max_tokens:
            return
        dev = self.wkv.device
        self.max_tokens = max_tokens
        self.staging = torch.zeros(max_tokens * self.rpt, self.row_bytes, dtype=torch.uint8, device=dev)
        self.rows = torch.zeros(max_tokens, self.rpt * self.dim, dtype=torch.bfloat16, device=dev)
        self.kv = torch.zeros(max_tokens, 5 * self.H, dtype=torch.bfloat16, device=dev)

    def forward(self, streams: torch.Tensor, rows_q_host, text_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """streams [T, 4, H] bf16 (updated in place), rows_q_host: uint8 [>= T * rows_per_token, row_bytes] (numpy or a
        pinned tensor, e.g. a gather slot), text_mask: device uint8 [>= T] or None.  Asynchronous on the current
        stream after the upload."""
        T = streams.shape[0]
        assert T <= self.max_tokens and streams.dtype == torch.bfloat16 and streams.is_contiguous()
        k, st = lib.kernels(), lib.stream
        src = rows_q_host if isinstance(rows_q_host, torch.Tensor) else torch.from_numpy(rows_q_host)
        n = T * self.rpt
        self.staging[:n].copy_(src[:n], non_blocking=True)
        if self.table_format == "nvfp4":
            lib.check(k.ds41_engram_dequant_nvfp4(lib.ptr(self.staging), self.row_bytes, self.dim,
                                                  C.c_float(self.table_scale), lib.ptr(self.rows), n, st()),
                      "engram_dequant_nvfp4")
        else:
            lib.check(k.ds41_engram_dequant(lib.ptr(self.staging), self.row_bytes, self.dim, lib.ptr(self.rows), n,
                                            st()), "engram_dequant")
        G.matmul_nt(self.rows[:T], self.wkv, self.kv[:T], status=self.status)
        lib.check(k.ds41_engram_gate(lib.ptr(streams), lib.ptr(self.kv), lib.ptr(self.q_w), lib.ptr(self.k_w),
                                     lib.ptr(text_mask), lib.ptr(streams), T, self.H, C.c_float(self.eps), st()),
                  "engram_gate")
        return streams

    def apply(self, streams: torch.Tensor, rows_q_host, text_mask: Optional[torch.Tensor] = None) -> None:
        """forward() for callers that expect no return value (the engine's launch wrapper); the projection's device
        status word is `self.status`."""
        self.forward(streams, rows_q_host, text_mask)


def init_engram_weights(hidden: int, rows_per_token: int = 24, row_dim: int = 256, seed: int = 0, std: float = 0.02):
    """Random Engram projection for tests and random-init models: (wkv [5H, rows_per_token * row_dim], q_weight [4, H],
    k_weight [4, H]) as fp32 CPU tensors."""
    g = torch.Generator().manual_seed(seed)
    wkv = torch.randn(5 * hidden, rows_per_token * row_dim, generator=g) * std
    q_w = 1.0 + 0.1 * torch.randn(4, hidden, generator=g)
    k_w = 1.0 + 0.1 * torch.randn(4, hidden, generator=g)
    return wkv, q_w, k_w


def random_table_rows(n_rows: int, row_dim: int = 256, row_bytes: int = 264, seed: int = 0) -> torch.Tensor:
    """A table of `n_rows` records in the checkpoint's row format (e4m3 payload + UE8M0 scale per 32, padded to
    `row_bytes`) with values of order one: uint8 [n_rows, row_bytes]."""
    g = torch.Generator().manual_seed(seed)
    vals = (torch.randn(n_rows, row_dim, generator=g)).clamp(-3, 3)
    out = torch.zeros(n_rows, row_bytes, dtype=torch.uint8)
    out[:, :row_dim] = vals.to(torch.float8_e4m3fn).view(torch.uint8)
    out[:, row_dim:row_dim + row_dim // 32] = torch.randint(125, 129, (n_rows, row_dim // 32), generator=g,
                                                            dtype=torch.int32).to(torch.uint8)
    return out
