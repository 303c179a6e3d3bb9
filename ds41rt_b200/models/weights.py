"""Random-initialised weights in the official tensor naming.

Names follow the official checkpoint templates (reference:
rust/crates/ds41rt-loader/src/official-v41-tensors.json): `embed.weight`,
`layers.{l}.attn.wq_a.weight`, `layers.{l}.ffn.experts.{e}.w1.weight`,
`mtp.{s}...`.  Here every tensor is fp32 (the oracle's dtype); GPU models
cast/quantise from this dict or generate large tensors directly on device.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config import ModelConfig


def _block_names(cfg: ModelConfig, prefix: str, layer_cfg: dict) -> Dict[str, tuple]:
    H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
    hpg = cfg.heads_per_group
    n_experts = layer_cfg["n_experts"]
    shapes = {
        f"{prefix}.attn_norm.weight": (H,),
        f"{prefix}.ffn_norm.weight": (H,),
        f"{prefix}.attn.wq_a.weight": (Q, H),
        f"{prefix}.attn.q_norm.weight": (Q,),
        f"{prefix}.attn.wq_b.weight": (cfg.n_heads * D, Q),
        f"{prefix}.attn.wkv.weight": (D, H),
        f"{prefix}.attn.kv_norm.weight": (D,),
        f"{prefix}.attn.wo_a.weight": (cfg.o_groups * cfg.o_lora, hpg * D),
        f"{prefix}.attn.wo_b.weight": (H, cfg.o_groups * cfg.o_lora),
        f"{prefix}.attn.attn_sink": (cfg.n_heads,),
        f"{prefix}.ffn.gate.weight": (n_experts, H),
        f"{prefix}.ffn.gate.bias": (n_experts,),
        f"{prefix}.ffn.shared_experts.w1.weight": (cfg.inter, H),
        f"{prefix}.ffn.shared_experts.w3.weight": (cfg.inter, H),
        f"{prefix}.ffn.shared_experts.w2.weight": (H, cfg.inter),
    }
    for kind in ("attn", "ffn"):
        shapes[f"{prefix}.hc_{kind}_fn"] = (cfg.hc_mult * 2 + cfg.hc_mult ** 2, cfg.hc_mult * H)
        shapes[f"{prefix}.hc_{kind}_scale"] = (3,)
        shapes[f"{prefix}.hc_{kind}_base"] = (cfg.hc_mult * 2 + cfg.hc_mult ** 2,)
    for e in range(n_experts):
        shapes[f"{prefix}.ffn.experts.{e}.w1.weight"] = (cfg.inter, H)
        shapes[f"{prefix}.ffn.experts.{e}.w3.weight"] = (cfg.inter, H)
        shapes[f"{prefix}.ffn.experts.{e}.w2.weight"] = (H, cfg.inter)
    return shapes


def tensor_shapes(cfg: ModelConfig, with_dspark: bool = True) -> Dict[str, tuple]:
    """name -> shape for every text-model tensor of `cfg` (vision/engram excluded)."""
    H, D = cfg.hidden, cfg.head_dim
    shapes: Dict[str, tuple] = {
        "embed.weight": (cfg.vocab, H),
        "head.weight": (cfg.vocab, H),
        "norm.weight": (H,),
    }
    for l in range(cfg.n_layers):
        p = f"layers.{l}"
        shapes.update(_block_names(cfg, p, {"n_experts": cfg.n_experts}))
        if l in cfg.source_layers:
            shapes[f"{p}.attn.compressor.wkv.weight"] = (D, H)
            shapes[f"{p}.attn.compressor.norm.weight"] = (D,)
            if cfg.source_layers[l] == 2:
                shapes[f"{p}.attn.compressor.wgate.weight"] = (D, H)
            shapes[f"{p}.attn.indexer.wk.weight"] = (cfg.index_dim, D)
            shapes[f"{p}.attn.indexer.k_norm.weight"] = (cfg.index_dim,)
        if l in cfg.index_layers:
            shapes[f"{p}.attn.indexer.wq_b.weight"] = (cfg.index_heads * cfg.index_dim, cfg.q_lora)
            shapes[f"{p}.attn.indexer.weights_proj.weight"] = (cfg.index_heads, H)
    if with_dspark and cfg.dspark is not None:
        d = cfg.dspark
        for s in range(d.stages):
            shapes.update(_block_names(cfg, f"mtp.{s}", {"n_experts": d.n_experts}))
        shapes["mtp.0.main_proj.weight"] = (H, H * len(d.tap_layers))
        shapes["mtp.0.main_norm.weight"] = (H,)
        last = d.stages - 1
        shapes[f"mtp.{last}.norm.weight"] = (H,)
        shapes[f"mtp.{last}.markov_head.embed.weight"] = (cfg.vocab, d.markov_rank)
        shapes[f"mtp.{last}.markov_head.head.weight"] = (cfg.vocab, d.markov_rank)
        shapes[f"mtp.{last}.confidence_head.proj.weight"] = (1, H + d.markov_rank)
    return shapes


def init_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02, with_dspark: bool = True,
                 device: str = "cpu") -> Dict[str, torch.Tensor]:
    """N(0, std) matrices (seeded, generated on CPU so every backend sees the
    same values), unit norm weights, and hyper-connection parameters chosen so the
    streams mix non-trivially."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg, with_dspark).items():
        if name.endswith("norm.weight"):
            t = torch.ones(shape)
        elif name.endswith("_scale"):
            t = torch.tensor([1.0, 1.0, 1.0])
        elif name.endswith("_base"):
            t = torch.randn(shape, generator=g) * 0.5
        elif name.endswith("_fn"):
            t = torch.randn(shape, generator=g) * std      # keeps the mixes' pre-activations O(1)
        elif name.endswith("attn_sink"):
            t = torch.randn(shape, generator=g) * 0.5
        elif name.endswith("gate.bias"):
            t = torch.randn(shape, generator=g) * 0.01
        else:
            t = torch.randn(shape, generator=g) * std
        out[name] = t.to(device)
    return out
