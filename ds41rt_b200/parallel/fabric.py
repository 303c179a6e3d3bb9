"""Peer-memory fabric: symmetric buffers every rank can load from / store to over NVLink.

One process per GPU.  `Fabric.create()` reads RANK/WORLD_SIZE, initialises torch.distributed (NCCL)
when world > 1 and hands out *symmetric* allocations: the same-sized buffer on every rank plus the
device pointers of all peers' copies, obtained through torch's symmetric-memory rendezvous
(CUDA VMM handles exchanged over the process group's store).  The fused kernels take those peer
pointers directly (P2P ld/st inside the kernel) together with bounded-spin flags that live in
symmetric memory too.  With world == 1 everything degenerates to local buffers.

Design parity: replaces the reference's coordinator<->worker transport and SM-issued peer copies
(native/cuda/kernels/v41_peer_copy.cu:6-80, rust/crates/ds41rt-transport/src/v41_expert/roce.rs:24-110).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class SymBuffer:
    local: torch.Tensor            # this rank's buffer (uint8 view base)
    peer_ptrs: List[int]           # device pointers of every rank's copy (index = rank)

    def view(self, dtype, shape, offset_bytes: int = 0) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes: offset_bytes + nbytes].view(dtype).view(*shape)


class Fabric:
    def __init__(self, rank: int, world: int, device: torch.device, group=None):
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self._keep = []

    # ------------------------------------------------------------------ construction
    @staticmethod
    def create(backend: str = "nccl") -> "Fabric":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            device = torch.device("cuda", local)
        else:
            device = torch.device("cpu")
        group = None
        if world > 1:
            import torch.distributed as dist
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29500")
                kw = {"device_id": device} if device.type == "cuda" else {}
                dist.init_process_group(backend=backend if device.type == "cuda" else "gloo", rank=rank,
                                        world_size=world, **kw)
            group = dist.group.WORLD
        return Fabric(rank, world, device, group)

    @staticmethod
    def single(device=None) -> "Fabric":
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        return Fabric(0, 1, torch.device(device), None)

    # ------------------------------------------------------------------ symmetric memory
    def alloc(self, nbytes: int) -> SymBuffer:
        nbytes = (nbytes + 255) // 256 * 256
        if self.world == 1:
            t = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            return SymBuffer(t, [t.data_ptr()])
        import torch.distributed._symmetric_memory as symm
        t = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm.rendezvous(t, self.group.group_name)
        t.zero_()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._keep.append(hdl)
        self.barrier()
        return SymBuffer(t, ptrs)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)

    def all_reduce_max(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def broadcast_object(self, obj, src: int = 0):
        if self.world == 1:
            return obj
        import torch.distributed as dist
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]
