"""GPU token sampler front end (csrc/kernels/sampler_rows.cu).

`sample_rows` draws one token per logits row with per-row parameters (temperature, top_k, top_p, min_p, seed,
position, allow-mask row).  The rule and the status codes are those of the host oracle `runtime.core.sample_token`
(reference: rust/crates/ds41rt-core/src/target_sampling.rs:180-243; GPU twin native/cuda/kernels/v41_sampling_gpu.cu).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import lib


@dataclass
class RowParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0
    position: int = 0
    mask_row: int = -1


def pack_params(params: Sequence[RowParams], device) -> torch.Tensor:
    """64-byte parameter blocks as a uint8 tensor on `device` (one host->device copy)."""
    arr = (lib.SampleRow * len(params))()
    for slot, p in zip(arr, params):
        slot.temperature, slot.top_k, slot.top_p, slot.min_p = p.temperature, p.top_k, p.top_p, p.min_p
        slot.seed, slot.position, slot.mask_row = p.seed & (2 ** 64 - 1), p.position, p.mask_row
    host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    return host.to(device)


def sample_rows(logits: torch.Tensor, params: torch.Tensor, masks: Optional[torch.Tensor] = None,
                tokens: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    """logits [rows, vocab] fp32 (row stride free), params from `pack_params`, masks [n, ceil(vocab/32)] int32/uint32.

    Returns (tokens int32 [rows], status int32 [rows]); asynchronous on the current stream."""
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    rows, vocab = logits.shape
    assert params.numel() == 64 * rows
    if tokens is None:
        tokens = torch.zeros(rows, dtype=torch.int32, device=logits.device)
    if status is None:
        status = torch.zeros(rows, dtype=torch.int32, device=logits.device)
    words = (vocab + 31) // 32
    if masks is not None:
        assert masks.dim() == 2 and masks.shape[1] == words and masks.is_contiguous()
    lib.check(lib.kernels().ds41_sample_rows(lib.ptr(logits), C.c_longlong(logits.stride(0)), rows, vocab, lib.ptr(masks),
                                             words, lib.ptr(params), lib.ptr(tokens), lib.ptr(status), lib.stream()),
              "sample_rows")
    return tokens, status
