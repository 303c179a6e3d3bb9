"""Scale-factor "atom" layout used by the block-scaled tensor-core GEMMs.

The MX kinds read one UE8M0 scale per 32 elements of K for every operand row.  tcgen05 wants them
in TMEM as [32 lanes] x [4 columns of 4 bytes]; the kernel copies 512-byte atoms there, one atom per
(128 rows, 128 elements of K):   byte offset = (row % 32) * 16 + ((row / 32) % 4) * 4 + (kblock % 4).
Atoms are stored row-atom major: [ceil(rows/128)][K/128][512].
"""
from __future__ import annotations

import torch


def pack_sf_atoms(e: torch.Tensor) -> torch.Tensor:
    """e: uint8 [rows, K/32] (K multiple of 128) -> uint8 [ceil(rows/128), K/128, 512]."""
    rows, kb = e.shape
    assert kb % 4 == 0
    ra = (rows + 127) // 128
    pad = torch.full((ra * 128, kb), 127, dtype=torch.uint8, device=e.device)
    pad[:rows] = e
    # [ra, 4 (row/32), 32 (row%32), ka, 4 (kb%4)] -> [ra, ka, 32, 4, 4]
    v = pad.view(ra, 4, 32, kb // 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return v.view(ra, kb // 4, 512)


def pack_sf_atoms_batched(e: torch.Tensor) -> torch.Tensor:
    """e: uint8 [batch, rows, K/32] -> uint8 [batch, ceil(rows/128), K/128, 512]; the same tiling as pack_sf_atoms for
    every batch entry in one pass (runs on whatever device `e` is on)."""
    b, rows, kb = e.shape
    assert kb % 4 == 0
    ra = (rows + 127) // 128
    pad = torch.full((b, ra * 128, kb), 127, dtype=torch.uint8, device=e.device)
    pad[:, :rows] = e
    v = pad.view(b, ra, 4, 32, kb // 4, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
    return v.view(b, ra, kb // 4, 512)


def unpack_sf_atoms(atoms: torch.Tensor, rows: int) -> torch.Tensor:
    ra, ka, _ = atoms.shape
    v = atoms.view(ra, ka, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(ra * 128, ka * 4)
    return v[:rows]
