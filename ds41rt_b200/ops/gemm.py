"""Python front end of the tcgen05 GEMM kernel (csrc/kernels/gemm_tc.cu).

All functions compute  D[m, n] = sum_k A[m, k] * B[n, k]  with both operands K-major
(i.e. `A @ B.T`).  For decode-sized inputs the weight matrix is passed as A and the few
token rows as B ("swap-AB") so the 128-row tensor-core tile is filled by weight rows;
the result is stored transposed, i.e. as [rows, features].
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import lib

KIND = {"bf16": 0, "fp8": 1, "mxfp8": 2}
_ELEM = {0: 2, 1: 1, 2: 1}


def pick_bn(rows: int) -> int:
    for bn in (16, 32, 64, 128):
        if rows <= bn:
            return bn
    return 128


def pick_splits(m: int, k: int, kind: int = 0, max_ctas: int = 148, max_splits: int = 16, n_tiles: int = 1,
                batch: int = 1) -> int:
    """Largest split-K factor that keeps the grid within one wave of `max_ctas` CTAs (no empty split)."""
    bk = 128 // _ELEM[kind]
    kb = (k + bk - 1) // bk
    tiles = ((m + 127) // 128) * n_tiles * batch
    s = max(1, min(max_splits, kb, max_ctas // max(tiles, 1)))
    while s > 1 and (s - 1) * ((kb + s - 1) // s) >= kb:
        s -= 1
    return s


def gemm_raw(A, B, out, M, N, K, *, lda, ldb, ldo, kind=0, out_mode=0, k_splits=1, bn=None, batch=1,
             a_batch_stride=0, b_batch_stride=0, out_batch_stride=0, a_batches=0, split_workspace=None,
             sfa=None, sfb=None, sfa_batch_stride=0, sfb_batch_stride=0, batch_map=None, n_active=None,
             b_batch_kind=0, up_row_offset=0, row_w=None, row_w_ld=0, act_limit=10.0, status=None,
             static_operand=0, a_format=0, col_limit=None, alpha=0.0, alpha_batch=None, signal=None):
    a = lib.GemmArgs()
    a.A, a.B, a.out = lib.ptr(A), lib.ptr(B), lib.ptr(out)
    a.split_workspace = lib.ptr(split_workspace)
    a.sfa, a.sfb = lib.ptr(sfa), lib.ptr(sfb)
    a.batch_map, a.n_active, a.row_w, a.status = lib.ptr(batch_map), lib.ptr(n_active), lib.ptr(row_w), lib.ptr(status)
    a.lda, a.ldb, a.ldo = lda, ldb, ldo
    a.a_batch_stride, a.b_batch_stride, a.out_batch_stride = a_batch_stride, b_batch_stride, out_batch_stride
    a.sfa_batch_stride, a.sfb_batch_stride = sfa_batch_stride, sfb_batch_stride
    a.M, a.N, a.K, a.batch, a.a_batches = M, N, K, batch, a_batches
    a.kind, a.out_mode, a.k_splits, a.bn = kind, out_mode, k_splits, bn or pick_bn(N)
    a.b_batch_kind, a.up_row_offset, a.row_w_ld, a.act_limit = b_batch_kind, up_row_offset, row_w_ld, act_limit
    a.static_operand = static_operand
    a.a_format = a_format
    a.col_limit = lib.ptr(col_limit)
    a.alpha = alpha
    a.alpha_batch = lib.ptr(alpha_batch)
    if signal is not None:          # (zeroed counter word, epoch word, device array of flag addresses, number of flags)
        a.sig_counter, a.sig_epoch, a.sig_flags, a.sig_world = (lib.ptr(signal[0]), lib.ptr(signal[1]),
                                                                lib.ptr(signal[2]), signal[3])
    lib.check(lib.kernels().ds41_gemm_tc(C.byref(a), lib.stream()), "ds41_gemm_tc")


def matmul_nt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, *, out_dtype=torch.bfloat16,
              status=None) -> torch.Tensor:
    """out[rows, N] = x[rows, K] @ w[N, K].T  (bf16 inputs).  Picks swap-AB for <= 128 rows."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
    rows, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        out = torch.empty(rows, N, dtype=out_dtype, device=x.device)
    f32 = out.dtype == torch.float32
    if rows <= 128:
        gemm_raw(w, x, out, N, rows, K, lda=w.stride(0), ldb=x.stride(0), ldo=out.stride(0),
                 out_mode=3 if f32 else 2, status=status, static_operand=1)
    else:
        # bf16 results leave through the TMA-store epilogue when the output rows are 16-byte aligned
        tma_out = not f32 and N >= 64 and (out.stride(0) * 2) % 16 == 0 and out.data_ptr() % 16 == 0
        gemm_raw(x, w, out, rows, N, K, lda=x.stride(0), ldb=w.stride(0), ldo=out.stride(0),
                 out_mode=1 if f32 else (6 if tma_out else 0), bn=256 if N >= 256 else (128 if N >= 128 else 64),
                 status=status, static_operand=2)
    return out


def linear_planes(x: torch.Tensor, w: torch.Tensor, planes: torch.Tensor, splits: int, *, status=None, signal=None):
    """Swap-AB split-K projection: planes[s, rows, N] (fp32) partial sums of x @ w.T.  `signal`: see gemm_raw."""
    rows, K = x.shape
    N = w.shape[0]
    assert planes.dtype == torch.float32 and planes.is_contiguous()
    if splits == 1:
        gemm_raw(w, x, planes, N, rows, K, lda=w.stride(0), ldb=x.stride(0), ldo=N, out_mode=3, status=status,
                 static_operand=1, signal=signal)
    else:
        gemm_raw(w, x, None, N, rows, K, lda=w.stride(0), ldb=x.stride(0), ldo=N, out_mode=3, k_splits=splits,
                 split_workspace=planes, status=status, static_operand=1, signal=signal)
