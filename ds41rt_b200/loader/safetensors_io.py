"""Strict safetensors container reader (and a small writer for tests / converted checkpoints).

Validation follows the reference loader (rust/crates/ds41rt-loader/src/v41_catalog.rs:566-662): known dtype, byte
length == prod(shape) * dtype size, data extents contiguous from offset 0, non-overlapping, and covering the data
section exactly (no trailing bytes).  Data is read through the native range reader (csrc/core/io.cc), including
row/column slices for tensor- and expert-parallel shards, with 64-bit offsets.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..ops import lib as _lib

# name -> (bits per element, torch dtype used to hold the raw payload)
DTYPES = {
    "BF16": (16, torch.bfloat16), "F16": (16, torch.float16), "F32": (32, torch.float32),
    "F8_E4M3": (8, torch.float8_e4m3fn), "F8_E8M0": (8, torch.uint8), "I8": (8, torch.int8), "U8": (8, torch.uint8),
    "I32": (32, torch.int32), "I64": (64, torch.int64), "F64": (64, torch.float64),
}
MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


@dataclass
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int      # offsets inside the data section
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file shorter than the header length field")
        with open(path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            if hlen > MAX_HEADER or 8 + hlen > size:
                raise SafetensorsError(f"{path}: header length {hlen} is implausible for a file of {size} bytes")
            raw = f.read(hlen)
        try:
            doc = json.loads(raw.decode("utf-8"))
        except Exception as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}")
        if not isinstance(doc, dict):
            raise SafetensorsError(f"{path}: header must be an object")
        self.metadata = doc.pop("__metadata__", {})
        self.data_start = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, d in doc.items():
            if not isinstance(d, dict) or set(d) != {"dtype", "shape", "data_offsets"}:
                raise SafetensorsError(f"{path}: malformed entry for '{name}'")
            dt, shape, offs = d["dtype"], d["shape"], d["data_offsets"]
            if dt not in DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype {dt}")
            if (not isinstance(shape, list) or any(not isinstance(x, int) or x < 0 for x in shape)
                    or not isinstance(offs, list) or len(offs) != 2 or any(not isinstance(x, int) for x in offs)):
                raise SafetensorsError(f"{path}: tensor '{name}' has a malformed shape or extent")
            n = 1
            for x in shape:
                n *= x
            want = n * DTYPES[dt][0] // 8
            if offs[1] - offs[0] != want or offs[0] < 0:
                raise SafetensorsError(f"{path}: tensor '{name}' extent {offs} does not match shape {shape} of {dt}")
            self.entries[name] = TensorEntry(name, dt, tuple(shape), offs[0], offs[1])
        cursor = 0
        for e in sorted(self.entries.values(), key=lambda e: (e.begin, e.end)):
            if e.begin != cursor:
                raise SafetensorsError(f"{path}: tensor '{e.name}' leaves a gap or overlaps at byte {cursor}")
            cursor = e.end
        if self.data_start + cursor != size:
            raise SafetensorsError(f"{path}: {size - self.data_start - cursor} trailing bytes after the last tensor")

    def names(self) -> List[str]:
        return list(self.entries)

    def read(self, name: str, rows: Optional[Tuple[int, int]] = None, cols: Optional[Tuple[int, int]] = None,
             threads: int = 4) -> torch.Tensor:
        """Whole tensor, or rows [r0,r1) and/or columns [c0,c1) of a 2-D tensor (element units)."""
        e = self.entries[name]
        bits, tdt = DTYPES[e.dtype]
        esz = bits // 8
        if len(e.shape) == 0 or (rows is None and cols is None):
            out = torch.empty(e.shape, dtype=tdt)
            rc = _lib.core().ds41_read_slice(self.path.encode(), C.c_uint64(self.data_start + e.begin),
                                             C.c_uint64(max(e.nbytes, 1)), C.c_uint64(0), C.c_uint64(1 if e.nbytes else 0),
                                             C.c_uint64(0), C.c_uint64(e.nbytes), C.c_void_p(out.data_ptr()), threads)
            if rc != 0:
                raise SafetensorsError(f"{self.path}: read of '{name}' failed ({rc})")
            return out
        if len(e.shape) != 2:
            lead = e.shape[0]
            inner = 1
            for x in e.shape[1:]:
                inner *= x
            if cols is not None:
                raise SafetensorsError("column slices need a 2-D tensor")
            shape2 = (lead, inner)
        else:
            shape2 = e.shape
        r0, r1 = rows if rows is not None else (0, shape2[0])
        c0, c1 = cols if cols is not None else (0, shape2[1])
        if not (0 <= r0 <= r1 <= shape2[0] and 0 <= c0 <= c1 <= shape2[1]):
            raise SafetensorsError(f"slice out of range for '{name}'")
        out_shape = (r1 - r0, c1 - c0) if len(e.shape) == 2 else (r1 - r0,) + tuple(e.shape[1:])
        out = torch.empty(out_shape, dtype=tdt)
        rc = _lib.core().ds41_read_slice(self.path.encode(), C.c_uint64(self.data_start + e.begin),
                                         C.c_uint64(shape2[1] * esz), C.c_uint64(r0), C.c_uint64(r1),
                                         C.c_uint64(c0 * esz), C.c_uint64(c1 * esz), C.c_void_p(out.data_ptr()), threads)
        if rc != 0:
            raise SafetensorsError(f"{self.path}: read of '{name}' failed ({rc})")
        return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], dtypes: Optional[Dict[str, str]] = None,
                      metadata: Optional[dict] = None):
    """Write tensors in insertion order.  `dtypes` overrides the container dtype name (e.g. F8_E8M0 for uint8)."""
    rev = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.float8_e4m3fn: "F8_E4M3",
           torch.uint8: "U8", torch.int8: "I8", torch.int32: "I32", torch.int64: "I64", torch.float64: "F64"}
    header, cursor, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        dt = (dtypes or {}).get(name, rev[t.dtype])
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [cursor, cursor + len(raw)]}
        cursor += len(raw)
        blobs.append(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
