"""Conversion between the official on-disk layout and the engine's name -> fp32 tensor dict.

`export_official` quantises an fp32 weight dict into the official layout (FP8+UE8M0 32x32 dense, FP4+UE8M0/32 routed
experts or the NVFP4 variant) and writes sharded safetensors + index; `load_official` reads a validated catalog back
into fp32 (dequantised) tensors, optionally only one rank's shard.  Used for small models and tests; the large-model
path streams shards straight into `EngineWeights` tensors.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..ops import quant_ref as Q
from .catalog import Catalog, expected_tensors
from .safetensors_io import write_safetensors


def _quantise(name: str, spec, w: Dict[str, torch.Tensor], variant: str):
    dt, shape = spec
    base, _, leaf = name.rpartition(".")
    if dt == "F8_E4M3" and leaf == "weight":
        if ".engram.embed" in name:                       # table rows carry one scale per 32 values of the row
            return Q.quant_mxfp8(w[name], 32)[0]
        q, _ = Q.quant_weight_mxfp8_32x32(w[name])
        return q
    if dt == "F8_E8M0" and leaf == "scale":
        src = w[base + ".weight"]
        if ".ffn.experts." in name:
            return Q.quant_mxfp4(src, 32)[1]
        if ".engram.embed" in name:
            return Q.quant_mxfp8(src, 32)[1]
        return Q.quant_weight_mxfp8_32x32(src)[1]
    if dt == "I8":
        return Q.quant_mxfp4(w[name], 32)[0].view(torch.int8)
    if dt == "U8" and leaf == "weight":
        return Q.quant_nvfp4(w[name])[0]
    if leaf == "weight_scale":
        return Q.quant_nvfp4(w[base + ".weight"])[1]
    if leaf == "weight_scale_2":
        return Q.quant_nvfp4(w[base + ".weight"])[2].reshape(())
    if leaf == "input_scale":
        return torch.tensor(1.0)
    t = w[name]
    return t.to(torch.bfloat16) if dt == "BF16" else t.to(torch.float32)


def export_official(cfg: ModelConfig, w: Dict[str, torch.Tensor], directory: str, variant: str = "mxfp4",
                    shards: int = 2, with_vision: bool = False, with_engram: bool = False):
    os.makedirs(directory, exist_ok=True)
    want = expected_tensors(cfg, variant, with_vision, with_engram)
    names = list(want)
    per = (len(names) + shards - 1) // shards
    weight_map = {}
    for s in range(shards):
        part = names[s * per:(s + 1) * per]
        if not part:
            continue
        fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        tensors, dts = {}, {}
        for n in part:
            if n.endswith("gate.bias_vl") and n not in w:
                t = torch.zeros(want[n][1])
            else:
                t = _quantise(n, want[n], w, variant)
            assert tuple(t.shape) == tuple(want[n][1]), (n, t.shape, want[n])
            tensors[n] = t
            dts[n] = want[n][0]
            weight_map[n] = fname
        write_safetensors(os.path.join(directory, fname), tensors, dts)
    json.dump({"metadata": {}, "weight_map": weight_map},
              open(os.path.join(directory, "model.safetensors.index.json"), "w"))


def load_official(cat: Catalog, rank: Optional[int] = None, world: int = 1) -> Dict[str, torch.Tensor]:
    """Dequantised fp32 tensors under the engine's names.  With `rank` given only that rank's shard is read
    (sliced tensors come back at their sliced shape)."""
    plan = cat.shard_plan(rank, world) if rank is not None else {n: (None, None) for n in cat.expected}
    out: Dict[str, torch.Tensor] = {}
    for name, (rows, cols) in plan.items():
        dt, _ = cat.expected[name]
        base, _, leaf = name.rpartition(".")
        if leaf in ("scale", "weight_scale", "weight_scale_2", "input_scale"):
            continue
        raw = cat.read(name, rows, cols)
        if dt == "F8_E4M3" and leaf == "weight":
            srows, scols = plan[base + ".scale"]
            e = cat.read(base + ".scale", srows, scols)
            if ".engram.embed" in name:
                out[name] = Q.dequant_mxfp8(raw, e, 32)
            else:
                out[name] = Q.dequant_weight_mxfp8_32x32(raw, e)
        elif dt == "I8":
            out[name] = Q.dequant_mxfp4(raw.view(torch.uint8), cat.read(base + ".scale", rows, None), 32)
        elif dt == "U8" and leaf == "weight":
            out[name] = Q.dequant_nvfp4(raw, cat.read(base + ".weight_scale", rows, None),
                                        cat.read(base + ".weight_scale_2").float())
        else:
            out[name] = raw.float()
    return out


class LazyOfficialWeights:
    """Mapping view of a validated checkpoint: a tensor is read and dequantised to fp32 when it is indexed, so a
    consumer that walks the model layer by layer never holds more than the tensors it is converting."""

    def __init__(self, cat: Catalog):
        self.cat = cat

    def expert_stack_fp4(self, prefix: str, e0: int, e1: int, device):
        """Routed experts [e0, e1) of the layer `prefix` ("layers.7", "mtp.0") in the engine's MX-FP4 layout, taken
        byte for byte from an FP4 + UE8M0/32 checkpoint: the E2M1 payloads are the checkpoint's bytes (w1 rows, then
        w3 rows), only the scales are re-tiled into the tensor cores' 128 x 4 atoms, on the device and for all experts
        at once.  No value is dequantised.  Returns (w13, w13 atoms, w2, w2 atoms), or None when the checkpoint holds
        another expert format.  (The reference re-tiles on the GPU too: native/cuda/kernels/v41_expert_pack.cu:10-107.)"""
        from ..ops.mx import pack_sf_atoms_batched
        cat = self.cat
        probe = f"{prefix}.ffn.experts.{e0}.w1.weight"
        if probe not in cat.expected or cat.expected[probe][0] != "I8":
            return None
        u8 = lambda name: cat.read(name).view(torch.uint8)
        w13, s13, w2, s2 = [], [], [], []
        for e in range(e0, e1):
            b = f"{prefix}.ffn.experts.{e}"
            w13.append(torch.cat([u8(f"{b}.w1.weight"), u8(f"{b}.w3.weight")], 0))
            s13.append(torch.cat([u8(f"{b}.w1.scale"), u8(f"{b}.w3.scale")], 0))
            w2.append(u8(f"{b}.w2.weight"))
            s2.append(u8(f"{b}.w2.scale"))
        up = lambda ts: torch.stack(ts).to(device, non_blocking=True).contiguous()
        return (up(w13), pack_sf_atoms_batched(up(s13)), up(w2), pack_sf_atoms_batched(up(s2)))

    def __contains__(self, name: str) -> bool:
        return name in self.cat.expected

    def __getitem__(self, name: str) -> torch.Tensor:
        cat = self.cat
        dt, _ = cat.expected[name]
        base, _, leaf = name.rpartition(".")
        raw = cat.read(name)
        if dt == "F8_E4M3" and leaf == "weight":
            e = cat.read(base + ".scale")
            return Q.dequant_mxfp8(raw, e, 32) if ".engram.embed" in name else Q.dequant_weight_mxfp8_32x32(raw, e)
        if dt == "I8":
            return Q.dequant_mxfp4(raw.view(torch.uint8), cat.read(base + ".scale"), 32)
        if dt == "U8" and leaf == "weight":
            return Q.dequant_nvfp4(raw, cat.read(base + ".weight_scale"), cat.read(base + ".weight_scale_2").float())
        return raw.float()


def load_engine_weights(directory: str, cfg: ModelConfig, rank: int, world: int, device, variant: str = "mxfp4",
                        expert_dtype: str = "mxfp8", with_vision: bool = False, with_engram: bool = False):
    """Validate the checkpoint under `directory` against the catalog and stream it into one rank's `EngineWeights`
    (reference: rust/crates/ds41rt-loader/src/v41_catalog.rs:478-637 for validation and range reads,
    v41_expert_staging for the per-rank expert plan)."""
    from ..models.ds41 import EngineWeights
    cat = Catalog(directory, cfg, variant, with_vision=with_vision, with_engram=with_engram)
    return EngineWeights.from_fp32(cfg, LazyOfficialWeights(cat), rank, world, device, expert_dtype=expert_dtype)


# ------------------------------------------------------------------------------------------------- Engram memory
def export_engram_table(cat: Catalog, layer: int, path: str, row_bytes: int = 264, chunk_rows: int = 1 << 20) -> int:
    """Write layer `layer`'s Engram table as the flat file the host gather maps: one record per table row,
    `head_dim` e4m3 bytes followed by head_dim/32 UE8M0 scale bytes, zero padded to `row_bytes`.  Streams the
    checkpoint in chunks of `chunk_rows` rows; returns the number of rows written.
    (Reference: rust/crates/ds41rt-loader/src/mapped_rows.rs:15 maps the same records.)"""
    name = f"layers.{layer}.engram.embed"
    _, (n_rows, dim) = cat.expected[name + ".weight"]
    assert dim + dim // 32 <= row_bytes
    with open(path, "wb") as f:
        for r0 in range(0, n_rows, chunk_rows):
            r1 = min(n_rows, r0 + chunk_rows)
            rec = torch.zeros(r1 - r0, row_bytes, dtype=torch.uint8)
            rec[:, :dim] = cat.read(name + ".weight", (r0, r1), None).view(torch.uint8)
            rec[:, dim:dim + dim // 32] = cat.read(name + ".scale", (r0, r1), None).view(torch.uint8)
            f.write(rec.numpy().tobytes())
    return n_rows


def load_engram_layer(directory: str, cfg: ModelConfig, layer: int, device, variant: str = "mxfp4",
                      table_format: str = "fp8", table_scale: float = 1.0):
    """The projection and gate weights of one Engram layer of an official checkpoint -> models.engram.EngramLayer
    (the table itself stays on the host: export_engram_table + runtime.engram.EngramPipeline)."""
    from ..models.engram import EngramLayer
    cat = Catalog(directory, cfg, variant, with_vision=False, with_engram=True)
    w = LazyOfficialWeights(cat)
    p = f"layers.{layer}.engram"
    bf = lambda t: t.to(device=device, dtype=torch.bfloat16).contiguous()
    g = cfg.engram
    return EngramLayer(bf(w[p + ".wkv.weight"]), bf(w[p + ".q_weight"]), bf(w[p + ".k_weight"]), cfg.hidden,
                       rows_per_token=g.n_heads * (g.max_ngram - 1), row_dim=g.head_dim, table_format=table_format,
                       table_scale=table_scale)
