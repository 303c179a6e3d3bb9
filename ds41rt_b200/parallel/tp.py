"""Tensor-parallel linear layers with the collective fused into the GEMM kernel.

Sequence-parallel layout: activations are sharded by rows across the ranks between blocks.
  * `ColumnParallelLinear` (all-gather -> GEMM): y[all rows, N_local] = gather(x) @ W_local^T.  The kernel's TMA
    producer fetches every peer's row tiles straight from that peer's symmetric buffer (no cluster multicast), starting
    with the local shard and walking the peers in ring order, after a bounded wait on each peer's "shard ready" flag -
    so the NVLink transfer of tile i+1 overlaps the tensor-core work on tile i.
  * `RowParallelLinear` (GEMM -> reduce-scatter): partial[all rows, N] = x[all rows, K_local] @ W[:, K_local]^T.  The
    epilogue stores each output tile directly into the owning rank's symmetric buffer (one slot per source rank);
    the owner sums the slots in rank order after a flag wait.
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
        # two alternating shard buffers: a peer may still be fetching call n while this rank prepares call n+1;
        # by the time call n+2 is written every peer has signalled n+1, i.e. has finished its GEMM of call n
        self.shard_bytes = rows_per_rank * self.K * 2
        self.x_sym = fabric.alloc(2 * self.shard_bytes)
        self._x = [self.x_sym.view(torch.bfloat16, (rows_per_rank, self.K), i * self.shard_bytes) for i in range(2)]
        self.parity = 0

    @property
    def x(self) -> torch.Tensor:
        """This rank's row shard for the NEXT forward call (write it on the current stream)."""
        return self._x[self.parity]

    def forward(self, out: torch.Tensor) -> torch.Tensor:
        """self.x holds this rank's row shard (written on the current stream).  out: [world*rows, N_local] bf16."""
        f, N = self.f, self.w.shape[0]
        self.flags.signal()
        a = lib.GemmArgs()
        a.B, a.out, a.status = lib.ptr(self.w), lib.ptr(out), lib.ptr(self.flags.status)
        a.lda, a.ldb, a.ldo = self.K, self.w.stride(0), out.stride(0)
        a.M, a.N, a.K, a.batch = f.world * self.rows, N, self.K, 1
        a.kind, a.out_mode, a.k_splits, a.bn = 0, 0, 1, 256 if N >= 256 else 128
        a.static_operand = 2
        a.ag_world, a.ag_rank, a.ag_rows = f.world, f.rank, self.rows
        for r in range(f.world):
            a.a_peers[r] = self.x_sym.peer_ptrs[r] + self.parity * self.shard_bytes
        a.ag_flags, a.ag_epoch = lib.ptr(self.flags.flag_ptrs), lib.ptr(self.flags.epoch)
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
        self.slot_bytes = fabric.world * rows_per_rank * self.N * 4
        self.slot_sym = fabric.alloc(2 * self.slot_bytes)           # alternating, same reasoning as the AG shards
        self._slots = [self.slot_sym.view(torch.float32, (fabric.world, rows_per_rank, self.N), i * self.slot_bytes)
                       for i in range(2)]
        self.parity = 0

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """x: [world*rows, K_local] bf16; out: [rows, N] bf16 = this rank's row shard of the summed product."""
        f = self.f
        a = lib.GemmArgs()
        a.A, a.B, a.status = lib.ptr(x), lib.ptr(self.w), lib.ptr(self.flags.status)
        a.lda, a.ldb, a.ldo = x.stride(0), self.w.stride(0), self.N
        a.M, a.N, a.K, a.batch = f.world * self.rows, self.N, self.K, 1
        a.kind, a.out_mode, a.k_splits, a.bn = 0, 1, 1, 256 if self.N >= 256 else 128
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
        lib.check(lib.kernels().ds41_rs_reduce(lib.ptr(slots), f.world, C.c_longlong(n), lib.ptr(out), 1,
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
