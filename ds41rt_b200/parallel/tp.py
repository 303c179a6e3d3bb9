"""Tensor-parallel linear layers with the collective fused into the GEMM kernel.

Sequence-parallel layout: activations are sharded by rows across the ranks between blocks.
  * `ColumnParallelLinear` (all-gather -> GEMM): y[all rows, N_local] = gather(x) @ W_local^T.  Two copier warps in
    every CTA of the GEMM push this rank's rows into every peer's copy of the gathered matrix (16-byte P2P stores,
    one arrival counter per source and 128-row tile); the TMA producer starts on the local rows and loads a remote
    tile from local memory as soon as its counter is complete - each byte crosses NVLink once and the transfer
    overlaps the tensor-core work.
  * `RowParallelLinear` (GEMM -> reduce-scatter): partial[all rows, N] = x[all rows, K_local] @ W[:, K_local]^T.  The
    epilogue stages bf16 tiles in shared memory and writes them with TMA stores straight into the owning rank's
    symmetric buffer (one slot per source rank, remote destinations first); the owner sums the slots in rank order
    after a flag wait.
A path that calls NCCL all_gather / reduce_scatter around a library matmul is kept as the baseline for comparison.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops import gemm as G
from ..ops import lib
from .fabric import Fabric


class SyncFlags:
    """One monotonically increasing epoch flag per rank in symmetric memory (see csrc/kernels/moe.cu signal_kernel)."""

    def __init__(self, fabric: Fabric):
        self.fabric = fabric
        self.sym = fabric.alloc(256)
        self.flag = self.sym.view(torch.int32, (1,), 0)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=fabric.device)
        self.flag_ptrs = torch.tensor(self.sym.peer_ptrs, dtype=torch.int64, device=fabric.device)
        self.status = lib.new_status(fabric.device)

    def signal(self):
        if self.fabric.world > 1:
            lib.check(lib.kernels().ds41_signal(lib.ptr(self.epoch), lib.ptr(self.flag), lib.stream()), "signal")


class ColumnParallelLinear:
    def __init__(self, fabric: Fabric, w_local: torch.Tensor, rows_per_rank: int, flags: Optional[SyncFlags] = None):
        assert rows_per_rank % 128 == 0 and w_local.dtype == torch.bfloat16
        self.f, self.w, self.rows = fabric, w_local, rows_per_rank
        self.K = w_local.shape[1]
        self.flags = flags or SyncFlags(fabric)
        self.calls = SyncFlags(fabric)          # private call counter: arrival targets are calls * chunks
        W = fabric.world
        # two alternating copies of the gathered matrix: a peer may already push call n+1 while this rank still
        # multiplies call n; call n+2 cannot start anywhere before every rank has finished call n
        self.full_bytes = W * rows_per_rank * self.K * 2
        self.x_sym = fabric.alloc(2 * self.full_bytes)
        self._full = [self.x_sym.view(torch.bfloat16, (W * rows_per_rank, self.K), i * self.full_bytes) for i in range(2)]
        self.arrive_sym = fabric.alloc(4 * W * (rows_per_rank // 128))
        self.parity = 0

    @property
    def x(self) -> torch.Tensor:
        """This rank's row shard for the NEXT forward call (write it on the current stream)."""
        r0 = self.f.rank * self.rows
        return self._full[self.parity][r0: r0 + self.rows]

    def forward(self, out: torch.Tensor) -> torch.Tensor:
        """self.x holds this rank's row shard (written on the current stream).  out: [world*rows, N_local] bf16."""
        f, N = self.f, self.w.shape[0]
        self.calls.signal()
        a = lib.GemmArgs()
        a.B, a.out, a.status = lib.ptr(self.w), lib.ptr(out), lib.ptr(self.flags.status)
        a.lda, a.ldb, a.ldo = self.K, self.w.stride(0), out.stride(0)
        a.M, a.N, a.K, a.batch = f.world * self.rows, N, self.K, 1
        a.kind, a.out_mode, a.k_splits, a.bn = 0, 6, 1, 256 if N >= 256 else 128
        a.static_operand = 2
        a.ag_world, a.ag_rank, a.ag_rows = f.world, f.rank, self.rows
        for r in range(f.world):
            a.a_peers[r] = self.x_sym.peer_ptrs[r] + self.parity * self.full_bytes
            a.ag_arrive[r] = self.arrive_sym.peer_ptrs[r]
        a.ag_epoch = lib.ptr(self.calls.epoch)
        lib.check(lib.kernels().ds41_gemm_tc(C.byref(a), lib.stream()), "ag_gemm")
        self.parity ^= 1
        return out

    def baseline(self, out: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        full = torch.empty(self.f.world * self.rows, self.K, dtype=torch.bfloat16, device=self.x.device)
        if self.f.world > 1:
            dist.all_gather_into_tensor(full, self.x, group=self.f.group)
        else:
            full.copy_(self.x)
        torch.matmul(full, self.w.t(), out=out)
        return out


class RowParallelLinear:
    def __init__(self, fabric: Fabric, w_local: torch.Tensor, rows_per_rank: int, flags: Optional[SyncFlags] = None):
        assert rows_per_rank % 128 == 0 and w_local.dtype == torch.bfloat16
        self.f, self.w, self.rows = fabric, w_local, rows_per_rank
        self.N, self.K = w_local.shape
        self.flags = flags or SyncFlags(fabric)
        self.slot_bytes = fabric.world * rows_per_rank * self.N * 2     # bf16 partial rows, one slot per source
        self.slot_sym = fabric.alloc(2 * self.slot_bytes)           # alternating, same reasoning as the AG shards
        self._slots = [self.slot_sym.view(torch.bfloat16, (fabric.world, rows_per_rank, self.N), i * self.slot_bytes)
                       for i in range(2)]
        self.parity = 0

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """x: [world*rows, K_local] bf16; out: [rows, N] bf16 = this rank's row shard of the summed product."""
        f = self.f
        a = lib.GemmArgs()
        a.A, a.B, a.status = lib.ptr(x), lib.ptr(self.w), lib.ptr(self.flags.status)
        a.lda, a.ldb, a.ldo = x.stride(0), self.w.stride(0), self.N
        a.M, a.N, a.K, a.batch = f.world * self.rows, self.N, self.K, 1
        a.kind, a.out_mode, a.k_splits, a.bn = 0, 6, 1, 256 if self.N >= 256 else 128
        a.static_operand = 2
        a.rs_world, a.rs_rank, a.rs_rows = f.world, f.rank, self.rows
        for r in range(f.world):
            a.rs_out[r] = self.slot_sym.peer_ptrs[r] + self.parity * self.slot_bytes
        lib.check(lib.kernels().ds41_gemm_tc(C.byref(a), lib.stream()), "gemm_rs")
        self.flags.signal()
        n = self.rows * self.N
        wait = lib.ptr(self.flags.flag_ptrs) if f.world > 1 else lib.ptr(None)
        slots = self._slots[self.parity]
        self.parity ^= 1
        lib.check(lib.kernels().ds41_rs_reduce(lib.ptr(slots), f.world, C.c_longlong(n), lib.ptr(out), 3,
                                               C.c_longlong(n), wait, lib.ptr(self.flags.epoch),
                                               lib.ptr(self.flags.status), lib.stream()), "rs_reduce")
        return out

    def baseline(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        full = torch.matmul(x, self.w.t())
        if self.f.world > 1:
            dist.reduce_scatter_tensor(out, full, group=self.f.group)
        else:
            out.copy_(full)
        return out
