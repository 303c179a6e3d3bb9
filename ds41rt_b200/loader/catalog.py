"""Official DeepSeek-V4.1 tensor catalog: expected names / dtypes / shapes, strict checkpoint validation and the
per-rank partition plan.

Layout (reference: rust/crates/ds41rt-loader/src/official-v41-tensors.json, v41_catalog.rs:393-441,478-637,699-758):
  * dense projections: `X.weight` F8_E4M3 [N, K] + `X.scale` F8_E8M0 [N/32, K/32] (one power-of-two scale per 32x32 tile)
  * routed experts:    `w{1,2,3}.weight` I8 [N, K/2] (two E2M1 values per byte, even element in the low nibble)
                       + `w{1,2,3}.scale` F8_E8M0 [N, K/32]
  * NVFP4 variant:     `weight` U8 [N, K/2] + `weight_scale` F8_E4M3 [N, K/16] + `weight_scale_2` F32 [] + `input_scale` F32 []
  * norms / gates / hyper-connection parameters in BF16 / F32.
Checkpoints are `model.safetensors.index.json` + shards; validation demands every expected tensor exactly once with
the exact dtype and shape and rejects unknown names.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

from ..config import ModelConfig
from .safetensors_io import SafetensorsError, SafetensorsFile

Spec = Tuple[str, Tuple[int, ...]]   # (dtype name, shape)


def _fp8(name: str, n: int, k: int, out: Dict[str, Spec]):
    out[f"{name}.weight"] = ("F8_E4M3", (n, k))
    out[f"{name}.scale"] = ("F8_E8M0", (n // 32, k // 32))


def _expert(prefix: str, cfg: ModelConfig, variant: str, out: Dict[str, Spec]):
    H, I = cfg.hidden, cfg.inter
    for w, (n, k) in (("w1", (I, H)), ("w3", (I, H)), ("w2", (H, I))):
        if variant == "nvfp4":
            out[f"{prefix}.{w}.weight"] = ("U8", (n, k // 2))
            out[f"{prefix}.{w}.weight_scale"] = ("F8_E4M3", (n, k // 16))
            out[f"{prefix}.{w}.weight_scale_2"] = ("F32", ())
            out[f"{prefix}.{w}.input_scale"] = ("F32", ())
        else:
            out[f"{prefix}.{w}.weight"] = ("I8", (n, k // 2))
            out[f"{prefix}.{w}.scale"] = ("F8_E8M0", (n, k // 32))


def _block(p: str, cfg: ModelConfig, n_experts: int, variant: str, out: Dict[str, Spec]):
    H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
    out[f"{p}.attn_norm.weight"] = ("BF16", (H,))
    out[f"{p}.ffn_norm.weight"] = ("BF16", (H,))
    _fp8(f"{p}.attn.wq_a", Q, H, out)
    out[f"{p}.attn.q_norm.weight"] = ("BF16", (Q,))
    _fp8(f"{p}.attn.wq_b", cfg.n_heads * D, Q, out)
    _fp8(f"{p}.attn.wkv", D, H, out)
    out[f"{p}.attn.kv_norm.weight"] = ("BF16", (D,))
    _fp8(f"{p}.attn.wo_a", cfg.o_groups * cfg.o_lora, cfg.heads_per_group * D, out)
    _fp8(f"{p}.attn.wo_b", H, cfg.o_groups * cfg.o_lora, out)
    out[f"{p}.attn.attn_sink"] = ("F32", (cfg.n_heads,))
    nproj = 2 * cfg.hc_mult + cfg.hc_mult ** 2
    for kind in ("attn", "ffn"):
        out[f"{p}.hc_{kind}_fn"] = ("F32", (nproj, cfg.hc_mult * H))
        out[f"{p}.hc_{kind}_scale"] = ("F32", (3,))
        out[f"{p}.hc_{kind}_base"] = ("F32", (nproj,))
    out[f"{p}.ffn.gate.weight"] = ("BF16", (n_experts, H))
    out[f"{p}.ffn.gate.bias"] = ("F32", (n_experts,))
    out[f"{p}.ffn.gate.bias_vl"] = ("F32", (n_experts,))
    for w, (n, k) in (("w1", (cfg.inter, H)), ("w3", (cfg.inter, H)), ("w2", (H, cfg.inter))):
        _fp8(f"{p}.ffn.shared_experts.{w}", n, k, out)
    for e in range(n_experts):
        _expert(f"{p}.ffn.experts.{e}", cfg, variant, out)


def expected_tensors(cfg: ModelConfig, variant: str = "mxfp4", with_vision: bool = True,
                     with_engram: bool = True) -> Dict[str, Spec]:
    """Every tensor of a checkpoint for `cfg` -> (dtype, shape)."""
    H, D = cfg.hidden, cfg.head_dim
    out: Dict[str, Spec] = {"embed.weight": ("BF16", (cfg.vocab, H)), "head.weight": ("BF16", (cfg.vocab, H)),
                            "norm.weight": ("BF16", (H,))}
    for l in range(cfg.n_layers):
        p = f"layers.{l}"
        _block(p, cfg, cfg.n_experts, variant, out)
        if l in cfg.source_layers:
            out[f"{p}.attn.compressor.wkv.weight"] = ("BF16", (D, H))
            out[f"{p}.attn.compressor.norm.weight"] = ("BF16", (D,))
            if cfg.source_layers[l] == 2:
                out[f"{p}.attn.compressor.wgate.weight"] = ("BF16", (D, H))
            out[f"{p}.attn.indexer.wk.weight"] = ("BF16", (cfg.index_dim, D))
            out[f"{p}.attn.indexer.k_norm.weight"] = ("BF16", (cfg.index_dim,))
        if l in cfg.index_layers:
            _fp8(f"{p}.attn.indexer.wq_b", cfg.index_heads * cfg.index_dim, cfg.q_lora, out)
            out[f"{p}.attn.indexer.weights_proj.weight"] = ("BF16", (cfg.index_heads, H))
        if with_engram and cfg.engram is not None and l in cfg.engram.layers:
            i = cfg.engram.layers.index(l)
            g = cfg.engram
            out[f"{p}.engram.embed.weight"] = ("F8_E4M3", (g.num_embeddings[i], g.head_dim))
            out[f"{p}.engram.embed.scale"] = ("F8_E8M0", (g.num_embeddings[i], g.head_dim // 32))
            out[f"{p}.engram.k_weight"] = ("BF16", (cfg.hc_mult, H))
            out[f"{p}.engram.q_weight"] = ("BF16", (cfg.hc_mult, H))
            width = (g.max_ngram - 1) * g.n_heads * g.head_dim
            _fp8(f"{p}.engram.wkv", (cfg.hc_mult + 1) * H, width, out)
    if cfg.dspark is not None:
        d = cfg.dspark
        for s in range(d.stages):
            _block(f"mtp.{s}", cfg, d.n_experts, variant, out)
        _fp8("mtp.0.main_proj", H, H * len(d.tap_layers), out)
        out["mtp.0.main_norm.weight"] = ("BF16", (H,))
        last = d.stages - 1
        out[f"mtp.{last}.norm.weight"] = ("BF16", (H,))
        out[f"mtp.{last}.markov_head.embed.weight"] = ("BF16", (cfg.vocab, d.markov_rank))
        out[f"mtp.{last}.markov_head.head.weight"] = ("BF16", (cfg.vocab, d.markov_rank))
        out[f"mtp.{last}.confidence_head.proj.weight"] = ("BF16", (1, H + d.markov_rank))
    if with_vision and cfg.vision is not None:
        v = cfg.vision
        W = v.hidden
        merged = W * v.downsample ** 2
        out.update({"aligner.w1.weight": ("BF16", (H, merged)), "aligner.w1.bias": ("BF16", (H,)),
                    "aligner.w2.weight": ("BF16", (H, H)), "aligner.w2.bias": ("BF16", (H,)),
                    "image_start": ("BF16", (H,)), "image_end": ("BF16", (H,)), "image_newline": ("BF16", (H,)),
                    "vision.norm.weight": ("BF16", (W,)),
                    "vision.patch_embed.proj.weight": ("BF16", (W, 3 * v.patch * v.patch)),
                    "vision.patch_embed.proj.bias": ("BF16", (W,))})
        for b in range(v.layers):
            p = f"vision.blocks.{b}"
            out.update({f"{p}.attn.wqkv.weight": ("BF16", (3 * W, W)), f"{p}.attn.wqkv.bias": ("BF16", (3 * W,)),
                        f"{p}.attn.wo.weight": ("BF16", (W, W)), f"{p}.attn.wo.bias": ("BF16", (W,)),
                        f"{p}.mlp.w1.weight": ("BF16", (2 * v.intermediate, W)),
                        f"{p}.mlp.w2.weight": ("BF16", (W, v.intermediate)),
                        f"{p}.norm1.weight": ("BF16", (W,)), f"{p}.norm2.weight": ("BF16", (W,))})
    return out


def official_templates(cfg: ModelConfig, variant: str = "mxfp4") -> List[str]:
    """Distinct name templates (layer / expert indices replaced by {}), e.g. 116 for the official Flash config."""
    import re
    seen = []
    for name, (dt, shape) in expected_tensors(cfg, variant).items():
        t = re.sub(r"(?<=\.)\d+(?=\.)", "{}", name)
        key = (t, dt, shape)
        if key not in seen:
            seen.append(key)
    return sorted({k[0] + "|" + k[1] + "|" + "x".join(map(str, k[2])) for k in seen})


@dataclass
class Located:
    file: SafetensorsFile
    name: str


class Catalog:
    """A validated checkpoint directory."""

    def __init__(self, directory: str, cfg: ModelConfig, variant: str = "mxfp4", with_vision: bool = True,
                 with_engram: bool = True):
        self.dir, self.cfg, self.variant = directory, cfg, variant
        index = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(index):
            doc = json.load(open(index))
            if "weight_map" not in doc or not isinstance(doc["weight_map"], dict):
                raise SafetensorsError("index has no weight_map")
            weight_map = doc["weight_map"]
        else:
            single = os.path.join(directory, "model.safetensors")
            if not os.path.exists(single):
                raise SafetensorsError(f"{directory}: neither an index nor model.safetensors found")
            weight_map = None
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, SafetensorsFile] = {}
        if weight_map is None:
            f = SafetensorsFile(single)
            self.files["model.safetensors"] = f
            for n in f.names():
                self.where[n] = f
        else:
            for name, shard in weight_map.items():
                if os.path.basename(shard) != shard:
                    raise SafetensorsError(f"index maps '{name}' outside the checkpoint directory")
                if shard not in self.files:
                    self.files[shard] = SafetensorsFile(os.path.join(directory, shard))
                if name not in self.files[shard].entries:
                    raise SafetensorsError(f"index places '{name}' in {shard}, which does not contain it")
                self.where[name] = self.files[shard]
            listed = sum(len(f.entries) for f in self.files.values())
            if listed != len(weight_map):
                raise SafetensorsError("shards contain tensors that the index does not list")
        want = expected_tensors(cfg, variant, with_vision, with_engram)
        missing = [n for n in want if n not in self.where]
        extra = [n for n in self.where if n not in want]
        if missing:
            raise SafetensorsError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:3]}")
        if extra:
            raise SafetensorsError(f"checkpoint has {len(extra)} unknown tensors, e.g. {extra[:3]}")
        for n, (dt, shape) in want.items():
            e = self.where[n].entries[n]
            if e.dtype != dt or tuple(e.shape) != tuple(shape):
                raise SafetensorsError(f"tensor '{n}' is {e.dtype}{list(e.shape)}, expected {dt}{list(shape)}")
        self.expected = want

    def read(self, name: str, rows=None, cols=None):
        return self.where[name].read(name, rows, cols)

    # ------------------------------------------------------------------ partition plan
    def shard_plan(self, rank: int, world: int) -> Dict[str, Tuple[Optional[Tuple[int, int]], Optional[Tuple[int, int]]]]:
        """name -> (row range, column range) this rank reads; replicated tensors map to (None, None).
        Attention heads / wo_a groups / shared-expert intermediate / vocabulary rows are sliced; routed experts are
        owned whole by one rank (expert parallel)."""
        cfg = self.cfg
        D = cfg.head_dim
        plan = {}
        HL, GL = cfg.n_heads // world, cfg.o_groups // world
        ISH, VL = cfg.inter // world, cfg.vocab // world
        for name in self.expected:
            rows = cols = None
            parts = name.split(".")
            if ".ffn.experts." in name:
                e = int(parts[parts.index("experts") + 1])
                n_exp = cfg.dspark.n_experts if name.startswith("mtp.") else cfg.n_experts
                if e // (n_exp // world) != rank:
                    continue
            elif name == "head.weight" or ".markov_head.head." in name:
                rows = (rank * VL, (rank + 1) * VL)
            elif name.endswith("attn.wq_b.weight") and ".indexer." not in name:
                rows = (rank * HL * D, (rank + 1) * HL * D)
            elif name.endswith("attn.wq_b.scale") and ".indexer." not in name:
                rows = (rank * HL * D // 32, (rank + 1) * HL * D // 32)
            elif name.endswith("attn.wo_a.weight"):
                rows = (rank * GL * cfg.o_lora, (rank + 1) * GL * cfg.o_lora)
            elif name.endswith("attn.wo_a.scale"):
                rows = (rank * GL * cfg.o_lora // 32, (rank + 1) * GL * cfg.o_lora // 32)
            elif name.endswith("attn.wo_b.weight"):
                cols = (rank * GL * cfg.o_lora, (rank + 1) * GL * cfg.o_lora)
            elif name.endswith("attn.wo_b.scale"):
                cols = (rank * GL * cfg.o_lora // 32, (rank + 1) * GL * cfg.o_lora // 32)
            elif name.endswith("attn.attn_sink"):
                rows = (rank * HL, (rank + 1) * HL)
            elif ".shared_experts.w1." in name or ".shared_experts.w3." in name:
                div = 32 if name.endswith(".scale") else 1
                rows = (rank * ISH // div, (rank + 1) * ISH // div)
            elif ".shared_experts.w2." in name:
                div = 32 if name.endswith(".scale") else 1
                cols = (rank * ISH // div, (rank + 1) * ISH // div)
            plan[name] = (rows, cols)
        return plan

    def shard_bytes(self, rank: int, world: int) -> int:
        total = 0
        for name, (rows, cols) in self.shard_plan(rank, world).items():
            e = self.where[name].entries[name]
            frac = 1.0
            if rows is not None and e.shape:
                frac *= (rows[1] - rows[0]) / max(e.shape[0], 1)
            if cols is not None and len(e.shape) > 1:
                frac *= (cols[1] - cols[0]) / max(e.shape[1], 1)
            total += int(e.nbytes * frac)
        return total
