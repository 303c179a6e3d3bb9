"""GPU execution of the DS41 architecture with the hand-written sm_100a kernels.

`DS41Engine` owns one rank's weight shards, caches and step buffers and enqueues one
"rows" pass (a decode step, a speculative verification chunk or a prefill chunk) as a fixed
sequence of kernel launches on the current stream - the sequence is CUDA-graph capturable
because every buffer is static and every data-dependent quantity (routes, selections, active
experts) stays on the device.

Parallel layout (world = tensor/expert-parallel degree on one NVSwitch box):
  * attention heads and wo_a groups sharded by rank, wo_b column-sharded -> fp32 partial planes
  * routed experts sharded by rank (EP), shared expert intermediate-sharded (TP) -> one partial plane
  * the partial planes live in symmetric memory; the next hyper-connection kernel sums every rank's
    plane with P2P loads in fixed rank order (deterministic one-shot all-reduce fused into the consumer)
  * vocabulary head row-sharded; greedy candidates merged through symmetric memory

Per-layer order of operations follows rust/crates/ds41rt-daemon/src/v41_backbone_execution.rs:615-677
and v41_hc.rs:153-225 (see models/reference.py for the mathematics).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig, rope_inv_freq
from ..ops import attention as A
from ..ops import gemm as G
from ..ops import lib
from ..parallel.fabric import Fabric, SymBuffer

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32


@dataclass
class LayerWeights:
    # hyper-connections
    hc_attn_fn: torch.Tensor = None
    hc_attn_scale: torch.Tensor = None
    hc_attn_base: torch.Tensor = None
    hc_ffn_fn: torch.Tensor = None
    hc_ffn_scale: torch.Tensor = None
    hc_ffn_base: torch.Tensor = None
    attn_norm: torch.Tensor = None
    ffn_norm: torch.Tensor = None
    # attention
    w_qkv: torch.Tensor = None          # [Q + D (+2D|D) (+IH), H]
    q_norm: torch.Tensor = None
    kv_norm: torch.Tensor = None
    w_qb: torch.Tensor = None           # [HL*D (+IH*ID), Q]
    wo_a: torch.Tensor = None           # [G_local, o_lora, hpg*D]
    wo_b: torch.Tensor = None           # [H, G_local*o_lora]
    sink: torch.Tensor = None
    # compressor / indexer
    comp_norm: Optional[torch.Tensor] = None
    wk_idx: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    # MoE
    w_gate_sh: torch.Tensor = None      # [E + 2*I_sh, H]
    gate_bias: torch.Tensor = None
    w2_sh: torch.Tensor = None          # [H, I_sh]
    w13: torch.Tensor = None            # [E_local, 2I, H]
    w2: torch.Tensor = None             # [E_local, H, I]
    w13_sf: Optional[torch.Tensor] = None   # MX experts: scale atoms [E_local, 2I/128, H/128, 512]
    w2_sf: Optional[torch.Tensor] = None    # [E_local, H/128, I/128, 512]
    # unsharded attention / shared-expert weights for sequence-parallel long passes (world > 1); where the layouts
    # allow it the rank's shards above are views of these
    w_qb_full: Optional[torch.Tensor] = None       # [n_heads*D (+IH*ID), Q]
    wo_a_full: Optional[torch.Tensor] = None       # [o_groups, o_lora, hpg*D]
    wo_b_full: Optional[torch.Tensor] = None       # [H, o_groups*o_lora]
    sink_full: Optional[torch.Tensor] = None       # [n_heads]
    w_gate_full: Optional[torch.Tensor] = None     # [E + 2*I, H]
    w2_sh_full: Optional[torch.Tensor] = None      # [H, I]
    n_experts: int = 0
    topk: int = 0
    extra_cols: int = 0
    index_heads_cols: int = 0
    ratio: int = 0                      # > 0: this layer produces a compressed source


def quantize_expert_stack(w: torch.Tensor, device):
    """[E, n, k] fp32 -> (E4M3 payload on device, scale atoms [E, n/128, k/128, 512]) with 128x128 power-of-two
    block scales expanded to the per-row / per-32 granularity of the MX tensor-core path."""
    from ..ops import quant_ref as Q
    from ..ops.mx import pack_sf_atoms
    qs, sfs = [], []
    for e in range(w.shape[0]):
        q, ex = Q.quant_weight_fp8_ue8m0_block(w[e], 128)
        qs.append(q)
        sfs.append(pack_sf_atoms(Q.expand_block_scales(ex, 128)))
    return torch.stack(qs).to(device).contiguous(), torch.stack(sfs).to(device).contiguous()


def quantize_expert_stack_fp4(w: torch.Tensor, device):
    """[E, n, k] fp32 -> (E2M1 codes two per byte [E, n, k/2], scale atoms [E, n/128, k/128, 512]): the official routed
    expert format (UE8M0 scale per 32 elements), consumed directly by the block-scaled GEMM with FP4 weights."""
    from ..ops import quant_ref as Q
    from ..ops.mx import pack_sf_atoms
    qs, sfs = [], []
    for e in range(w.shape[0]):
        q, ex = Q.quant_mxfp4(w[e], 32)
        qs.append(q)
        sfs.append(pack_sf_atoms(ex))
    return torch.stack(qs).to(device).contiguous(), torch.stack(sfs).to(device).contiguous()


def dequantize_expert_fp4(q: torch.Tensor, sf_atoms: torch.Tensor) -> torch.Tensor:
    from ..ops import quant_ref as Q
    from ..ops.mx import unpack_sf_atoms
    return Q.dequant_mxfp4(q.cpu(), unpack_sf_atoms(sf_atoms.cpu(), q.shape[0]), 32)


def quantize_expert_stack_nvfp4(w: torch.Tensor, device):
    """[E, n, k] fp32 -> (e2m1 codes two per byte [E, n, k/2], E4M3 scale atoms [E, n/128, k/64, 512], global scales [E]):
    the NVFP4 W4A4 expert variant (one E4M3 scale per 16 elements and one fp32 scale per tensor)."""
    from ..ops import quant_ref as Q
    from ..ops.mx import pack_sf_atoms
    qs, sfs, gs = [], [], []
    for e in range(w.shape[0]):
        q, bs, g = Q.quant_nvfp4(w[e])
        qs.append(q)
        sfs.append(pack_sf_atoms(bs.view(torch.uint8)))
        gs.append(float(g))
    return (torch.stack(qs).to(device).contiguous(), torch.stack(sfs).to(device).contiguous(),
            torch.tensor(gs, dtype=torch.float32, device=device))


def dequantize_expert_nvfp4(q: torch.Tensor, sf_atoms: torch.Tensor, gs: float) -> torch.Tensor:
    from ..ops import quant_ref as Q
    from ..ops.mx import unpack_sf_atoms
    bs = unpack_sf_atoms(sf_atoms.cpu(), q.shape[0]).view(torch.float8_e4m3fn)
    return Q.dequant_nvfp4(q.cpu(), bs, gs)


# fixed per-tensor scales of the NVFP4 activations (ModelOpt's input_scale): FC1 sees normalised hidden rows, FC2 the
# clamped SwiGLU output times the route weight
NVFP4_IN_SCALE_FC1 = 16.0 / (448.0 * 6.0)
NVFP4_IN_SCALE_FC2 = 8.0 / (448.0 * 6.0)


def dequantize_expert(q: torch.Tensor, sf_atoms: torch.Tensor) -> torch.Tensor:
    """Inverse of quantize_expert_stack for one expert (used by tests to feed the oracle)."""
    from ..ops import quant_ref as Q
    from ..ops.mx import unpack_sf_atoms
    e = unpack_sf_atoms(sf_atoms.cpu(), q.shape[0])
    return Q.dequant_mxfp8(q.cpu(), e)


class EngineWeights:
    """One rank's shard of the model in kernel layout."""
    expert_dtype = "bf16"

    def __init__(self, cfg: ModelConfig, rank: int, world: int, device):
        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        self.layers: List[LayerWeights] = []
        self.embed = None
        self.head = None           # [V_local, H]
        self.final_norm = None
        assert cfg.n_heads % world == 0 and cfg.o_groups % world == 0 and cfg.n_experts % world == 0
        assert cfg.vocab % world == 0 and cfg.inter % world == 0
        self.HL = cfg.n_heads // world
        self.GL = cfg.o_groups // world
        self.I_sh = cfg.inter // world
        self.V_local = cfg.vocab // world

    @staticmethod
    def from_fp32(cfg: ModelConfig, w: Dict[str, torch.Tensor], rank: int, world: int, device,
                  prefix: str = "layers", n_layers: Optional[int] = None, n_experts: Optional[int] = None,
                  topk: Optional[int] = None, expert_dtype: str = "bf16", share: Optional["EngineWeights"] = None,
                  layer_range: Optional[tuple] = None, full_dense: bool = True) -> "EngineWeights":
        """Build one rank's shard from an fp32 name->tensor dict.  expert_dtype "mxfp8" stores routed
        experts as E4M3 with power-of-two 128x128 block scales (consumed by the block-scaled GEMM).
        full_dense (world > 1): also keep the unsharded attention / shared-expert weights, which the sequence-parallel
        long pass multiplies against its own rows (about 0.3 GB per Flash layer in bf16)."""
        ew = EngineWeights(cfg, rank, world, device)
        ew.expert_dtype = expert_dtype
        D, H = cfg.head_dim, cfg.hidden
        dev = lambda t, dt=BF16: t.to(device=device, dtype=dt).contiguous()
        if share is not None:          # drafter blocks reuse the target's embedding and vocabulary head
            ew.embed, ew.head = share.embed, share.head
        else:
            ew.embed = dev(w["embed.weight"])
            v0 = rank * ew.V_local
            ew.head = dev(w["head.weight"][v0:v0 + ew.V_local])
        ew.final_norm = dev(w["norm.weight"], F32)
        n_layers = cfg.n_layers if n_layers is None else n_layers
        E = cfg.n_experts if n_experts is None else n_experts
        k = cfg.topk if topk is None else topk
        assert E % world == 0
        EL = E // world
        h0, h1 = rank * ew.HL, (rank + 1) * ew.HL
        g0, g1 = rank * ew.GL, (rank + 1) * ew.GL
        for l in range(n_layers):
            if layer_range is not None and not (layer_range[0] <= l < layer_range[1]):
                ew.layers.append(None)        # a pipeline stage holds only its own layers
                continue
            p = f"{prefix}.{l}"
            lw = LayerWeights(n_experts=E, topk=k)
            for kind in ("attn", "ffn"):
                setattr(lw, f"hc_{kind}_fn", dev(w[f"{p}.hc_{kind}_fn"], F32))
                setattr(lw, f"hc_{kind}_scale", dev(w[f"{p}.hc_{kind}_scale"], F32))
                setattr(lw, f"hc_{kind}_base", dev(w[f"{p}.hc_{kind}_base"], F32))
            lw.attn_norm = dev(w[f"{p}.attn_norm.weight"], F32)
            lw.ffn_norm = dev(w[f"{p}.ffn_norm.weight"], F32)
            parts = [w[f"{p}.attn.wq_a.weight"], w[f"{p}.attn.wkv.weight"]]
            extra = 0
            is_source = prefix == "layers" and l in cfg.source_layers
            is_index = prefix == "layers" and l in cfg.index_layers
            if is_source:
                lw.ratio = cfg.source_layers[l]
                parts.append(w[f"{p}.attn.compressor.wkv.weight"])
                extra += D
                if lw.ratio == 2:
                    parts.append(w[f"{p}.attn.compressor.wgate.weight"])
                    extra += D
                lw.comp_norm = dev(w[f"{p}.attn.compressor.norm.weight"], F32)
                lw.wk_idx = dev(w[f"{p}.attn.indexer.wk.weight"])
                lw.k_norm = dev(w[f"{p}.attn.indexer.k_norm.weight"], F32)
            if is_index:
                parts.append(w[f"{p}.attn.indexer.weights_proj.weight"])
                extra += cfg.index_heads
                lw.index_heads_cols = cfg.index_heads
            lw.extra_cols = extra
            lw.w_qkv = dev(torch.cat(parts, 0))
            lw.q_norm = dev(w[f"{p}.attn.q_norm.weight"], F32)
            lw.kv_norm = dev(w[f"{p}.attn.kv_norm.weight"], F32)
            qb = [w[f"{p}.attn.wq_b.weight"][h0 * D:h1 * D]]
            if is_index:
                qb.append(w[f"{p}.attn.indexer.wq_b.weight"])
            lw.w_qb = dev(torch.cat(qb, 0))
            wo_a = w[f"{p}.attn.wo_a.weight"].view(cfg.o_groups, cfg.o_lora, cfg.heads_per_group * D)
            i0, i1 = rank * ew.I_sh, (rank + 1) * ew.I_sh
            if world > 1 and full_dense:
                lw.w_qb_full = dev(torch.cat([w[f"{p}.attn.wq_b.weight"]] + qb[1:], 0))
                lw.wo_a_full = dev(wo_a)
                lw.wo_b_full = dev(w[f"{p}.attn.wo_b.weight"])
                lw.sink_full = dev(w[f"{p}.attn.attn_sink"], F32)
                lw.w_gate_full = dev(torch.cat([w[f"{p}.ffn.gate.weight"], w[f"{p}.ffn.shared_experts.w1.weight"],
                                                w[f"{p}.ffn.shared_experts.w3.weight"]], 0))
                lw.w2_sh_full = dev(w[f"{p}.ffn.shared_experts.w2.weight"])
                lw.wo_a = lw.wo_a_full[g0:g1]
                lw.wo_b = lw.wo_b_full[:, g0 * cfg.o_lora:g1 * cfg.o_lora]
                lw.sink = lw.sink_full[h0:h1]
                lw.w2_sh = lw.w2_sh_full[:, i0:i1]
            else:
                lw.wo_a = dev(wo_a[g0:g1])
                lw.wo_b = dev(w[f"{p}.attn.wo_b.weight"][:, g0 * cfg.o_lora:g1 * cfg.o_lora])
                lw.sink = dev(w[f"{p}.attn.attn_sink"][h0:h1], F32)
                lw.w2_sh = dev(w[f"{p}.ffn.shared_experts.w2.weight"][:, i0:i1])
            lw.w_gate_sh = dev(torch.cat([w[f"{p}.ffn.gate.weight"], w[f"{p}.ffn.shared_experts.w1.weight"][i0:i1],
                                          w[f"{p}.ffn.shared_experts.w3.weight"][i0:i1]], 0))
            lw.gate_bias = dev(w[f"{p}.ffn.gate.bias"], F32)
            if world == 1:
                lw.w_qb_full, lw.wo_a_full, lw.wo_b_full, lw.sink_full = lw.w_qb, lw.wo_a, lw.wo_b, lw.sink
                lw.w_gate_full, lw.w2_sh_full = lw.w_gate_sh, lw.w2_sh
            e0 = rank * EL
            raw = w.expert_stack_fp4(p, e0, e0 + EL, device) \
                if expert_dtype == "mxfp4" and hasattr(w, "expert_stack_fp4") else None
            if raw is not None:
                # an FP4 checkpoint into FP4 engine experts: bytes are copied, only the scales are re-tiled
                lw.w13, lw.w13_sf, lw.w2, lw.w2_sf = raw
                ew.layers.append(lw)
                continue
            w13 = torch.stack([torch.cat([w[f"{p}.ffn.experts.{e}.w1.weight"],
                                          w[f"{p}.ffn.experts.{e}.w3.weight"]], 0) for e in range(e0, e0 + EL)], 0)
            w2 = torch.stack([w[f"{p}.ffn.experts.{e}.w2.weight"] for e in range(e0, e0 + EL)], 0)
            if expert_dtype == "mxfp8":
                lw.w13, lw.w13_sf = quantize_expert_stack(w13, device)
                lw.w2, lw.w2_sf = quantize_expert_stack(w2, device)
            elif expert_dtype == "mxfp4":
                lw.w13, lw.w13_sf = quantize_expert_stack_fp4(w13, device)
                lw.w2, lw.w2_sf = quantize_expert_stack_fp4(w2, device)
            elif expert_dtype == "nvfp4":
                lw.w13, lw.w13_sf, lw.w13_gs = quantize_expert_stack_nvfp4(w13, device)
                lw.w2, lw.w2_sf, lw.w2_gs = quantize_expert_stack_nvfp4(w2, device)
            else:
                lw.w13, lw.w2 = dev(w13), dev(w2)
            ew.layers.append(lw)
        return ew

    @staticmethod
    def random(cfg: ModelConfig, rank: int, world: int, device, seed: int = 0, std: float = 0.02,
               router_std: Optional[float] = None, expert_dtype: str = "bf16",
               share: Optional["EngineWeights"] = None, layer_range: Optional[tuple] = None,
               full_dense: bool = True) -> "EngineWeights":
        """Random-init shard generated directly on the device (for models too large to stage on the host).
        expert_dtype "mxfp8": E4M3 payloads ~ N(0, 48^2) with every 128x128 block scale 2^-11 (dequantised
        std 0.0234), the statistics an amax-scaled quantisation of N(0, 0.02) weights produces."""
        ew = EngineWeights(cfg, rank, world, device)
        ew.expert_dtype = expert_dtype
        D, H, Q = cfg.head_dim, cfg.hidden, cfg.q_lora
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
        shared_gen = torch.Generator(device=device).manual_seed(seed * 1000 + 999)   # replicated tensors

        def rnd(shape, g=gen, s=std, dt=BF16):
            chunk = torch.empty(shape, dtype=dt, device=device)
            flat = chunk.view(-1)
            step = 1 << 26
            for i in range(0, flat.numel(), step):
                n = min(step, flat.numel() - i)
                flat[i:i + n] = (torch.randn(n, generator=g, device=device, dtype=F32) * s).to(dt)
            return chunk

        ones = lambda n: torch.ones(n, dtype=F32, device=device)
        if share is not None:
            ew.embed, ew.head = share.embed, share.head
        else:
            ew.embed = rnd((cfg.vocab, H), shared_gen)
            ew.head = rnd((ew.V_local, H))
        ew.final_norm = ones(H)
        EL = cfg.n_experts // world
        nproj = 2 * cfg.hc_mult + cfg.hc_mult ** 2
        for l in range(cfg.n_layers):
            if layer_range is not None and not (layer_range[0] <= l < layer_range[1]):
                ew.layers.append(None)        # a pipeline stage holds only its own layers
                continue
            lw = LayerWeights(n_experts=cfg.n_experts, topk=cfg.topk)
            for kind in ("attn", "ffn"):
                setattr(lw, f"hc_{kind}_fn", rnd((nproj, cfg.hc_mult * H), shared_gen, std, F32))
                setattr(lw, f"hc_{kind}_scale", ones(3))
                setattr(lw, f"hc_{kind}_base", rnd((nproj,), shared_gen, 0.5, F32))
            lw.attn_norm, lw.ffn_norm = ones(H), ones(H)
            extra = 0
            if l in cfg.source_layers:
                lw.ratio = cfg.source_layers[l]
                extra += D * (2 if lw.ratio == 2 else 1)
                lw.comp_norm = ones(D)
                lw.wk_idx = rnd((cfg.index_dim, D), shared_gen)
                lw.k_norm = ones(cfg.index_dim)
            if l in cfg.index_layers:
                extra += cfg.index_heads
                lw.index_heads_cols = cfg.index_heads
            lw.extra_cols = extra
            lw.w_qkv = rnd((Q + D + extra, H), shared_gen)
            lw.q_norm, lw.kv_norm = ones(Q), ones(D)
            n_idx = cfg.index_heads * cfg.index_dim if l in cfg.index_layers else 0
            E_g, I_all = cfg.n_experts, cfg.inter
            if world > 1 and full_dense:
                # the same unsharded tensors on every rank (replicated generator); the rank's shards are slices of them
                lw.w_qb_full = rnd((cfg.n_heads * D + n_idx, Q), shared_gen)
                lw.w_qb = torch.cat([lw.w_qb_full[rank * ew.HL * D:(rank + 1) * ew.HL * D],
                                     lw.w_qb_full[cfg.n_heads * D:]], 0).contiguous()
                lw.wo_a_full = rnd((cfg.o_groups, cfg.o_lora, cfg.heads_per_group * D), shared_gen)
                lw.wo_b_full = rnd((H, cfg.o_groups * cfg.o_lora), shared_gen)
                lw.sink_full = rnd((cfg.n_heads,), shared_gen, 0.5, F32)
                lw.w_gate_full = rnd((E_g + 2 * I_all, H), shared_gen)
                if router_std is not None:
                    lw.w_gate_full[:E_g] = rnd((E_g, H), shared_gen, router_std / math.sqrt(H) * 1.0)
                lw.w2_sh_full = rnd((H, I_all), shared_gen)
                i0, i1 = rank * ew.I_sh, (rank + 1) * ew.I_sh
                lw.wo_a = lw.wo_a_full[rank * ew.GL:(rank + 1) * ew.GL]
                lw.wo_b = lw.wo_b_full[:, rank * ew.GL * cfg.o_lora:(rank + 1) * ew.GL * cfg.o_lora]
                lw.sink = lw.sink_full[rank * ew.HL:(rank + 1) * ew.HL]
                lw.w_gate_sh = torch.cat([lw.w_gate_full[:E_g], lw.w_gate_full[E_g + i0:E_g + i1],
                                          lw.w_gate_full[E_g + I_all + i0:E_g + I_all + i1]], 0).contiguous()
                lw.w2_sh = lw.w2_sh_full[:, i0:i1]
            else:
                lw.w_qb = rnd((ew.HL * D + n_idx, Q))
                lw.wo_a = rnd((ew.GL, cfg.o_lora, cfg.heads_per_group * D))
                lw.wo_b = rnd((H, ew.GL * cfg.o_lora))
                lw.sink = rnd((ew.HL,), gen, 0.5, F32)
                lw.w_gate_sh = rnd((cfg.n_experts + 2 * ew.I_sh, H), shared_gen)
                if router_std is not None:
                    lw.w_gate_sh[:cfg.n_experts] = rnd((cfg.n_experts, H), shared_gen, router_std / math.sqrt(H) * 1.0)
                lw.w2_sh = rnd((H, ew.I_sh))
                if world == 1:
                    lw.w_qb_full, lw.wo_a_full, lw.wo_b_full, lw.sink_full = lw.w_qb, lw.wo_a, lw.wo_b, lw.sink
                    lw.w_gate_full, lw.w2_sh_full = lw.w_gate_sh, lw.w2_sh
            lw.gate_bias = rnd((cfg.n_experts,), shared_gen, 0.01, F32)
            if expert_dtype == "mxfp8":
                def rnd8(shape):
                    out = torch.empty(shape, dtype=torch.float8_e4m3fn, device=device)
                    flat = out.view(-1)
                    step = 1 << 26
                    for i in range(0, flat.numel(), step):
                        n = min(step, flat.numel() - i)
                        flat[i:i + n] = (torch.randn(n, generator=gen, device=device, dtype=F32) * 48.0).clamp(
                            -448, 448).to(torch.float8_e4m3fn)
                    return out
                I = cfg.inter
                lw.w13 = rnd8((EL, 2 * I, H))
                lw.w2 = rnd8((EL, H, I))
                lw.w13_sf = torch.full((EL, 2 * I // 128, H // 128, 512), 127 - 11, dtype=torch.uint8, device=device)
                lw.w2_sf = torch.full((EL, H // 128, I // 128, 512), 127 - 11, dtype=torch.uint8, device=device)
            elif expert_dtype == "nvfp4":
                # uniform random E2M1 codes, every 1x16 scale 1.0 (E4M3 0x38) and a global scale of 0.008 per expert:
                # dequantised std about 0.02
                def rnd4n(shape):
                    out = torch.empty(shape, dtype=torch.uint8, device=device)
                    flat = out.view(-1)
                    step = 1 << 27
                    for i in range(0, flat.numel(), step):
                        n = min(step, flat.numel() - i)
                        flat[i:i + n] = torch.randint(0, 256, (n,), generator=gen, device=device, dtype=torch.uint8)
                    return out
                I = cfg.inter
                lw.w13 = rnd4n((EL, 2 * I, H // 2))
                lw.w2 = rnd4n((EL, H, I // 2))
                lw.w13_sf = torch.full((EL, 2 * I // 128, H // 64, 512), 0x38, dtype=torch.uint8, device=device)
                lw.w2_sf = torch.full((EL, H // 128, I // 64, 512), 0x38, dtype=torch.uint8, device=device)
                lw.w13_gs = torch.full((EL,), 0.008, dtype=F32, device=device)
                lw.w2_gs = torch.full((EL,), 0.008, dtype=F32, device=device)
            elif expert_dtype == "mxfp4":
                # uniform random E2M1 codes (two per byte) with every 1x32 scale 2^-7: dequantised std about 0.024
                def rnd4(shape):
                    out = torch.empty(shape, dtype=torch.uint8, device=device)
                    flat = out.view(-1)
                    step = 1 << 27
                    for i in range(0, flat.numel(), step):
                        n = min(step, flat.numel() - i)
                        flat[i:i + n] = torch.randint(0, 256, (n,), generator=gen, device=device, dtype=torch.uint8)
                    return out
                I = cfg.inter
                lw.w13 = rnd4((EL, 2 * I, H // 2))
                lw.w2 = rnd4((EL, H, I // 2))
                lw.w13_sf = torch.full((EL, 2 * I // 128, H // 128, 512), 127 - 7, dtype=torch.uint8, device=device)
                lw.w2_sf = torch.full((EL, H // 128, I // 128, 512), 127 - 7, dtype=torch.uint8, device=device)
            else:
                lw.w13 = rnd((EL, 2 * cfg.inter, H))
                lw.w2 = rnd((EL, H, cfg.inter))
            ew.layers.append(lw)
        return ew

    def nbytes(self) -> int:
        """Bytes held by this rank (a storage shared by a tensor and its views counts once)."""
        seen, total = set(), 0
        ts = [self.embed, self.head, self.final_norm]
        for lw in self.layers:
            if lw is not None:
                ts += [v for v in vars(lw).values() if isinstance(v, torch.Tensor)]
        for t in ts:
            st = t.untyped_storage()
            if st.data_ptr() not in seen:
                seen.add(st.data_ptr())
                total += st.nbytes()
        return total


@dataclass
class KVSnapshot:
    """State of one request after `n_tokens` positions: enough to continue it in another slot.

    Full pages of the compressed / index pools are shared by reference (they are never written again); the rows of the
    last, partly filled page, the window rings of every layer and the ratio-2 pair carry are copied."""
    n_tokens: int
    pages: List[int]
    partial: Dict[int, tuple]
    rings: torch.Tensor
    pending: Dict[int, torch.Tensor]

    def nbytes(self) -> int:
        n = self.rings.numel() * self.rings.element_size()
        for a, b in self.partial.values():
            n += a.numel() * a.element_size() + b.numel() * b.element_size()
        return n + sum(t.numel() * t.element_size() for t in self.pending.values())


class KVCache:
    """Window rings, paged compressed pools and the page table for `slots` concurrent requests.

    A page covers `page_tokens` token positions; a source with compress ratio r stores
    page_tokens / r rows per page, so every source shares one page table
    (sizing rule: native counterpart rust/crates/ds41rt-daemon/src/v41_native_serve/memory.rs:9-13,137)."""

    def __init__(self, cfg: ModelConfig, n_layers: int, slots: int, max_ctx: int, device, page_tokens: int = 64,
                 n_pages: Optional[int] = None, spec_slack: int = 16, kv_dtype: str = "bf16",
                 index_dtype: Optional[str] = None):
        self.cfg, self.slots, self.max_ctx, self.page_tokens = cfg, slots, max_ctx, page_tokens
        assert kv_dtype in ("bf16", "fp8", "fp4")
        self.kv_dtype = kv_dtype
        # index keys: "fp4" = E2M1 pairs + one UE8M0 scale per 32 values (68 bytes per key of 128 values instead of
        # 256; the queries are then quantised the same way before the dot - the reference's FP4 x FP4 contract,
        # native/cuda/kernels/v41_index_scores.cu:36-103, v41_compressor.cu:25-57).  Default: FP4 with the FP4 cache.
        if index_dtype is None:
            index_dtype = "fp4" if kv_dtype == "fp4" and cfg.index_dim % 32 == 0 else "bf16"
        assert index_dtype in ("bf16", "fp4") and (index_dtype == "bf16" or cfg.index_dim % 32 == 0)
        self.index_dtype = index_dtype
        self.idx_row_bytes = (cfg.index_dim // 2 + cfg.index_dim // 32 + 3) // 4 * 4 if index_dtype == "fp4" else 0
        # FP8 rows: D e4m3 values + D/32 UE8M0 scales (per 32 elements), padded to 16 bytes; 0 = bf16 rows
        self.row_bytes = 0 if kv_dtype == "bf16" else (cfg.head_dim + cfg.head_dim // 32 + 15) // 16 * 16
        # "fp4": the window rings stay FP8, the compressed rows are FP4 (D/2 e2m1 bytes + D/16 E4M3 scales, the
        # reference's 288-byte rows for D = 512); 0 = compressed rows in the window's format
        self.comp_row_bytes = (cfg.head_dim // 2 + cfg.head_dim // 16 + 15) // 16 * 16 if kv_dtype == "fp4" else 0
        D = cfg.head_dim
        ring = cfg.window + spec_slack
        self.ring = ring
        self.max_pages = (max_ctx + page_tokens - 1) // page_tokens
        self.n_pages = n_pages if n_pages is not None else self.max_pages * slots
        kv_shape, kv_dt = ((D,), BF16) if self.row_bytes == 0 else ((self.row_bytes,), torch.uint8)
        self.win = torch.zeros(n_layers, slots, ring, *kv_shape, dtype=kv_dt, device=device)
        self.comp: Dict[int, torch.Tensor] = {}
        self.idx: Dict[int, torch.Tensor] = {}
        self.pending: Dict[int, torch.Tensor] = {}
        self.page_rows: Dict[int, int] = {}
        for src, ratio in cfg.source_layers.items():
            if src >= n_layers:
                continue
            pr = page_tokens // ratio
            self.page_rows[src] = pr
            comp_shape = (self.comp_row_bytes,) if self.comp_row_bytes else kv_shape
            self.comp[src] = torch.zeros(self.n_pages * pr, *comp_shape, dtype=kv_dt, device=device)
            self.idx[src] = (torch.zeros(self.n_pages * pr, self.idx_row_bytes, dtype=torch.uint8, device=device)
                             if self.idx_row_bytes else
                             torch.zeros(self.n_pages * pr, cfg.index_dim, dtype=BF16, device=device))
            if ratio == 2:
                self.pending[src] = torch.zeros(slots, 4, 2 * D, dtype=F32, device=device)
        self.page_table_host = torch.full((slots, self.max_pages), -1, dtype=I32)
        self.page_table = self.page_table_host.to(device)
        # Pages, reference counts and slot leases live in the host runtime's allocator (csrc/core/kvalloc.cc); this
        # class only mirrors each slot's page list into the device page table.
        from ..runtime import core as K
        self.alloc = K.KvAllocator(self.n_pages, slots, page_tokens)

    # ------------------------------------------------------------------ slots and pages
    @property
    def free_pages(self) -> int:
        return self.alloc.free_pages

    def pages_of(self, slot: int) -> List[int]:
        return self.alloc.pages(slot)

    def admit(self):
        """Lease a free slot -> (slot, generation), or None when every slot is taken."""
        return self.alloc.admit()

    def _gen(self, slot: int) -> int:
        """Generation of the slot's lease; a slot used without admit() (single-request drivers) is leased here."""
        g = self.alloc.generation(slot)
        if g == 0:
            g = self.alloc.admit_slot(slot)
            assert g is not None
        return g

    def _publish(self, slot: int, first: int = 0):
        pages = self.alloc.pages(slot)
        n = len(pages)
        if n > first:
            self.page_table_host[slot, first:n] = torch.tensor(pages[first:], dtype=I32)
            self.page_table[slot, first:n].copy_(self.page_table_host[slot, first:n], non_blocking=True)

    def ensure(self, slot: int, n_tokens: int) -> bool:
        """Make sure `slot` has pages for positions [0, n_tokens).  Returns False when the pool is exhausted."""
        need = (n_tokens + self.page_tokens - 1) // self.page_tokens
        if need > self.max_pages:
            return False
        gen = self._gen(slot)
        have = self.alloc.page_count(slot)
        if need <= have:
            return True
        try:
            self.alloc.ensure(slot, gen, n_tokens)
        except MemoryError:
            return False
        self._publish(slot, have)
        return True

    def release(self, slot: int):
        g = self.alloc.generation(slot)
        if g:
            self.alloc.retire(slot, g)
        self.page_table_host[slot].fill_(-1)
        self.page_table[slot].fill_(-1)

    # ------------------------------------------------------------------ prefix snapshots
    def snapshot(self, slot: int, n_tokens: int) -> KVSnapshot:
        """Capture `slot` after positions [0, n_tokens) (call it between passes, on the engine's stream)."""
        full = n_tokens // self.page_tokens
        mine = self.alloc.pages(slot)
        pages = self.alloc.retain(slot, self._gen(slot), min(full, len(mine)))
        partial = {}
        rem = n_tokens - full * self.page_tokens
        if rem and full < len(mine):
            pg = mine[full]
            for src, pr in self.page_rows.items():
                rows = (rem * pr + self.page_tokens - 1) // self.page_tokens
                partial[src] = (self.comp[src][pg * pr: pg * pr + rows].clone(), self.idx[src][pg * pr: pg * pr + rows].clone())
        return KVSnapshot(n_tokens, pages, partial, self.win[:, slot].clone(),
                          {src: t[slot].clone() for src, t in self.pending.items()})

    def restore_prefix(self, slot: int, snap: KVSnapshot, n_tokens: int) -> bool:
        """Give an empty `slot` the compressed / index rows of the snapshot's first `n_tokens` positions (an even
        count below the snapshot's length): whole pages below the cut are shared, the page the cut falls into is copied
        up to the cut.  Window rings and the pair carry are NOT restored: the caller replays the tokens from the cut on
        with a window floor at the cut.  Returns False when no page is free for the copied page."""
        gen = self._gen(slot)
        assert self.alloc.page_count(slot) == 0, "restore needs an empty slot"
        assert 0 < n_tokens <= snap.n_tokens and n_tokens % 2 == 0
        full = n_tokens // self.page_tokens
        rem = n_tokens - full * self.page_tokens
        if rem and self.alloc.free_pages == 0:
            return False
        self.alloc.share(slot, gen, snap.pages[:full])
        if rem:
            self.alloc.ensure(slot, gen, n_tokens)
            pg = self.alloc.pages(slot)[full]
            for src, pr in self.page_rows.items():
                rows = (rem * pr + self.page_tokens - 1) // self.page_tokens
                if full < len(snap.pages):                  # the cut falls into one of the snapshot's whole pages
                    sp = snap.pages[full]
                    c, ix = self.comp[src][sp * pr: sp * pr + rows], self.idx[src][sp * pr: sp * pr + rows]
                else:                                       # ... or into its partly filled last page
                    c, ix = snap.partial[src][0][:rows], snap.partial[src][1][:rows]
                self.comp[src][pg * pr: pg * pr + rows].copy_(c)
                self.idx[src][pg * pr: pg * pr + rows].copy_(ix)
        self._publish(slot)
        return True

    def restore(self, slot: int, snap: KVSnapshot) -> bool:
        """Continue a snapshot in an empty `slot`: shared full pages, a private copy of the partial page, rings and
        carry.  Returns False when no page is free for the partial page."""
        gen = self._gen(slot)
        assert self.alloc.page_count(slot) == 0, "restore needs an empty slot"
        if snap.partial and self.alloc.free_pages == 0:
            return False
        self.alloc.share(slot, gen, snap.pages)
        if snap.partial:
            self.alloc.ensure(slot, gen, (len(snap.pages) + 1) * self.page_tokens)
            pg = self.alloc.pages(slot)[len(snap.pages)]
            for src, (c, ix) in snap.partial.items():
                pr = self.page_rows[src]
                self.comp[src][pg * pr: pg * pr + c.shape[0]].copy_(c)
                self.idx[src][pg * pr: pg * pr + ix.shape[0]].copy_(ix)
        self._publish(slot)
        self.win[:, slot].copy_(snap.rings)
        for src, t in snap.pending.items():
            self.pending[src][slot].copy_(t)
        return True

    def drop_snapshot(self, snap: KVSnapshot):
        if snap.pages:
            self.alloc.release_pages(snap.pages)
        snap.pages = []

    def nbytes(self) -> int:
        ts = [self.win] + list(self.comp.values()) + list(self.idx.values()) + list(self.pending.values())
        return sum(t.numel() * t.element_size() for t in ts)


class DS41Engine:
    def __init__(self, cfg: ModelConfig, weights: EngineWeights, fabric: Optional[Fabric] = None, *,
                 max_rows: int = 8, slots: int = 1, max_ctx: int = 4096, page_tokens: int = 64,
                 n_pages: Optional[int] = None, row_hi: bool = False, moe_rows: int = 32, kv_dtype: str = "bf16",
                 long_pass: str = "auto", index_dtype: Optional[str] = None):
        """long_pass: how passes longer than `moe_rows` rows run on several ranks.  "sp" (sequence parallel): every rank
        owns rows/world rows of the residual streams; hyper-connections, q_b, indexer, attention over all heads, wo_a /
        wo_b, router and shared expert run on the own rows against unsharded weights, the normalised rows are
        all-gathered inside the q_a / kv projection (every rank writes every cache row) and the routed experts go
        through the all-to-all.  "replicated": every rank holds all rows, heads and shared expert are sharded and the
        partial planes are summed by peer reads.  "auto": "sp" where a pass allows it (rows a multiple of 128 x world,
        unsharded weights present, no Engram layer live), else "replicated"."""
        assert long_pass in ("auto", "sp", "replicated")
        self.long_pass = long_pass
        self.cfg, self.w = cfg, weights
        self.fabric = fabric or Fabric.single(weights.device)
        self.rank, self.world = self.fabric.rank, self.fabric.world
        self.device = dev = weights.device
        self.max_rows = R = max_rows
        self.n_layers = len(weights.layers)
        H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
        self.k = lib.kernels()
        # the window ring holds one pass of new rows beyond the window: a row still needs the key at pos - window + 1
        # after the last row of its pass has been written
        self.cache = KVCache(cfg, self.n_layers, slots, max_ctx, dev, page_tokens, n_pages, spec_slack=max(16, R),
                             kv_dtype=kv_dtype, index_dtype=index_dtype)
        self.HL, self.GL, self.I_sh, self.V_local = weights.HL, weights.GL, weights.I_sh, weights.V_local
        live = [lw for lw in weights.layers if lw is not None]      # a pipeline stage holds a slice of the stack
        self._lw_any = live[0] if live else None
        E = live[0].n_experts if live else cfg.n_experts
        self.E, self.topk = E, (live[0].topk if live else cfg.topk)
        self.EL = E // self.world
        # passes of at most moe_rows rows run every active expert over all rows (decode); longer passes sort the rows
        # by expert and go through the expert-parallel tile-table path (prefill)
        self.moe_rows = Rm = min(R, moe_rows)
        self.max_active = min(Rm * self.topk, self.EL)
        self._ep = None
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
        # inputs
        self.in_tokens = z((R,), I32)
        self.row_pos = z((R,), I32)
        self.row_slot = z((R,), I32)
        self.row_hi = z((R,), I32) if row_hi else None
        # residual state
        self.streams = z((R, cfg.hc_mult, H), BF16)
        self.pre = [z((R, 4), F32), z((R, 4), F32)]
        self.post = z((R, 4), F32)
        self.comb = z((R, 16), F32)
        self.n_slices = H // 128
        self.hc_partial = z((self.n_slices, R, 25), F32)
        self.xn = z((R, H), BF16)
        self.coef = [(z((R, 4), F32), z((R, 16), F32)), (z((R, 4), F32), z((R, 16), F32))]
        self.step_partial = z((self.n_slices, R, 26), F32)
        self.xc = z((R, H), F32)
        self.tickets = z((R,), I32)
        self.fused_rows = 16      # passes of at most this many rows use the fused hyper-connection step
        # Passes of at least `mix_tc_rows` rows take the 24 mixes projections of a hyper-connection step from a
        # tensor-core GEMM over the stored streams (mixing matrix as bf16 high + low parts) instead of SIMT dot products.
        self.mix_tc_rows = 128
        self._mix_w: Dict[int, torch.Tensor] = {}          # data_ptr of an fp32 mixing matrix -> [64, 4H] bf16 split
        self.mix_planes = z((max(R, 148 * 128) * 64,), F32) if R >= self.mix_tc_rows else None
        self._mix_state = None                             # (splits, rows) of the projection that hc_finish reads next
        self.taps = z((len(cfg.dspark.tap_layers), R, H), F32) if cfg.dspark is not None else None
        # attention
        max_extra = max([lw.extra_cols for lw in live] + [0])
        self.ntot_qkv = Q + D + max_extra
        self.max_splits = 16
        # layers differ in their extra columns; fewer columns can mean more splits, so size for every distinct width
        widths = sorted({lw.w_qkv.shape[0] for lw in live} | {self.ntot_qkv})
        self.planes_qkv = z((max(self._plane_rows(n) * n for n in widths),), F32)
        self.q_lat = z((R, Q), BF16)
        self.extras = z((R, max(max_extra, 1)), F32)
        self.nqb = self.HL * D + cfg.index_heads * cfg.index_dim
        self.qb_out = z((R, self.nqb), BF16)
        self.max_keys = max_ctx
        self.scores = z((R, self.max_keys), F32)
        if R > self.moe_rows and cfg.index_layers:
            self.idx_q = z((R * cfg.index_heads, cfg.index_dim), BF16)      # RoPE'd index queries, (row, head) major
            self.idx_k = z((self.max_keys, cfg.index_dim), BF16)            # one request's index keys, contiguous
            self.idx_vis = z((R,), I32)
        self.sel = z((R, cfg.index_topk), I32)
        self.n_sel = z((R,), I32)
        self.row_lo = z((R,), I32)      # window floor per row (set_rows(row_lo=...)); used only while _floor_on
        self._floor_on = False
        # candidate blocks: the candidate layer's block selection (list + bit mask per row) restricts the index layers
        # above it (reference: native/cuda/kernels/v41_candidate_blocks.cu:18-44)
        self.cand_on = cfg.candidate_layer >= 0 and cfg.candidate_topk_blocks > 0 and cfg.candidate_layer < self.n_layers
        if self.cand_on:
            nb = (self.max_keys + cfg.candidate_block - 1) // cfg.candidate_block
            self.cand_words = (nb + 31) // 32
            self.cand_mask = z((R, self.cand_words), I32)
            self.cand_blocks = z((R, cfg.candidate_topk_blocks), I32)
            self.cand_count = z((R,), I32)
        self._cand_ratio = None     # ratio of the source the live candidate mask was computed on (None = no mask)
        self.n_splits_attn = (cfg.window + 16 + cfg.index_topk + 63) // 64
        cells = max(r * self._attn_splits(r) for r in range(1, R + 1))      # (row, split) partial outputs
        self.part_o = z((cells, self.HL, D), F32)
        self.part_ml = z((cells, self.HL, 2), F32)
        self.attn_out = z((R, self.HL * D), BF16)
        self.oa = z((R, self.GL * cfg.o_lora), BF16)
        self.planes_oa = z((self.max_splits * self.GL * min(R, 16) * cfg.o_lora,), F32)    # split-K partials of wo_a
        # MoE
        self.ntot_gate = E + 2 * self.I_sh
        self.planes_gate = z((self._plane_rows(self.ntot_gate), self.ntot_gate), F32)
        self.ids = z((R, self.topk), I32)
        self.route_w = z((R, self.topk), F32)
        self.shared_act = z((R, self.I_sh), BF16)
        self.active = z((self.max_active,), I32)
        self.n_active = z((1,), I32)
        self.row_w = z((self.max_active, Rm), F32)
        self.slot_of = z((R, self.topk), I32)
        self.act = z((self.max_active, Rm, cfg.inter), BF16)
        self.nv = weights.expert_dtype == "nvfp4"         # W4A4: e2m1 weights and activations, E4M3 scales per 16
        self.mx = weights.expert_dtype in ("mxfp8", "mxfp4")
        self.a_fmt = 1 if weights.expert_dtype == "mxfp4" else 0     # routed expert weights in E2M1 (two per byte)
        if self.mx:
            assert H % 128 == 0 and cfg.inter % 128 == 0
            ra = (Rm + 127) // 128
            self.xq = z((R, H), torch.uint8)
            self.xq_sf = z(((R + 127) // 128, H // 128, 512), torch.uint8)
            self.actq = z((self.max_active, Rm, cfg.inter), torch.uint8)
            self.actq_sf = z((self.max_active, ra, cfg.inter // 128, 512), torch.uint8)
        if self.nv:
            assert H % 256 == 0 and cfg.inter % 256 == 0
            ra = (Rm + 127) // 128
            self.xq4 = z((R, H // 2), torch.uint8)
            self.xq4_sf = z(((R + 127) // 128, H // 64, 512), torch.uint8)
            self.actq4 = z((self.max_active, Rm, cfg.inter // 2), torch.uint8)
            self.actq4_sf = z((self.max_active, ra, cfg.inter // 64, 512), torch.uint8)
        self.fc2 = z((self.max_active, Rm, H), F32)
        self.planes_shared = z((self._plane_rows(H), H), F32)
        # head
        # long passes (prefill) only need the last row's logits: the head runs on at most head_cap rows
        self.head_cap = 64
        self.last_head_row = 0
        self.logits = z((min(R, self.head_cap), self.V_local), F32)
        self.chosen = z((R,), I32)
        self.status = lib.new_status(dev)
        # symmetric buffers: [attn planes | moe plane | flag | best_val | best_idx]
        o_rows = self._plane_rows(H)
        self.o_plane_bytes = o_rows * H * 4
        self.moe_plane_bytes = R * H * 4
        off_flag = self.o_plane_bytes + self.moe_plane_bytes
        off_best = off_flag + 256
        total = off_best + 2 * R * 4 + 256
        self.sym: SymBuffer = self.fabric.alloc(total)
        self.planes_o = self.sym.view(F32, (o_rows, H), 0)
        self.moe_plane = self.sym.view(F32, (R, H), self.o_plane_bytes)
        # flag area: one slot per rank; rank r publishes into slot r of EVERY rank's area, so waits poll local memory
        self.flag = self.sym.view(torch.int32, (max(self.world, 1),), off_flag)
        self.best_val = self.sym.view(F32, (R,), off_best)
        self.best_idx = self.sym.view(I32, (R,), off_best + R * 4)
        self.epoch = z((1,), I32)
        peers = self.sym.peer_ptrs
        self._o_bases = (C.c_void_p * self.world)(*[p for p in peers])
        self._moe_bases = (C.c_void_p * self.world)(*[p + self.o_plane_bytes for p in peers])
        self._val_ptrs = (C.c_void_p * self.world)(*[p + off_best for p in peers])
        self._idx_ptrs = (C.c_void_p * self.world)(*[p + off_best + R * 4 for p in peers])
        self.flag_ptrs = torch.tensor([peers[self.rank] + off_flag + 4 * r for r in range(self.world)],
                                      dtype=torch.int64, device=dev)           # where this rank waits: its own area
        self.flag_out = torch.tensor([p + off_flag + 4 * self.rank for p in peers], dtype=torch.int64, device=dev)
        self.sig_counters = z((2,), I32)          # arrival counters of the kernels that fold the publication in
        self._sig_attn = (self.sig_counters[0:1], self.epoch, self.flag_out, self.world) if self.world > 1 else None
        # rope tables
        self.inv_plain = torch.tensor(rope_inv_freq(cfg.rope_plain, cfg.rope_dim), dtype=F32, device=dev)
        self.inv_long = torch.tensor(rope_inv_freq(cfg.rope_long, cfg.rope_dim), dtype=F32, device=dev)
        self.inv_idx = torch.tensor(rope_inv_freq(cfg.rope_long, cfg.index_dim // 2), dtype=F32, device=dev)
        self.layer_prefix_plain = False   # drafter blocks use the plain rope
        self.launches = 0
        self.only = None
        from ..utils.trace import ActivationTrace
        self.layer_timer = None   # utils.trace.LayerTimer: device time per layer of eager passes
        # DS41_NVTX=1: every launch sits in an NVTX range named after its kernel class (for timeline tools)
        import os
        self.nvtx = os.environ.get("DS41_NVTX", "") == "1"
        self.activation_trace = ActivationTrace.from_env()
        self._pass_hint = None    # (rows, highest position) of a single-request pass described by the last set_rows
        self.image_patch = None   # (image rows, pass-row ids) applied after the embedding lookup of the next pass
        self.timeline = None   # set to a list to record (tag, start event, end event) per launch of eager passes
        # Engram memory layers: layer -> (EngramLayer, pinned host rows [max_rows * rows_per_token, row_bytes], device
        # text mask [max_rows] uint8).  A layer takes part in a pass only after set_engram_rows() filled its host rows.
        self.engram: Dict[int, tuple] = {}
        self._engram_live: set = set()
        self._engram_copied: Dict[int, object] = {}      # layer -> event after the last upload of its host rows
        self._engram_layer_of: Dict[int, int] = {}
        if R > self.moe_rows and live:
            self._make_ep(live[0])
        self.debug = None   # set to a list to record per-layer routing / selection decisions
        self.head_mask = None     # optional allow-mask rows for the greedy selection of every pass (see head_rows)
        self._sp = None           # buffers of the sequence-parallel long pass (made on first use)
        self._sp_ag = {}          # rows per rank -> all-gather context of the q_a / kv projection
        self._sp_active = None    # (first own row, own rows, rows) while the streams are row-sharded
        self._sp_pending = None   # (plane address, splits, split stride) of the own rows' unmerged sublayer

    # ------------------------------------------------------------------ helpers
    def _inv(self, layer: int) -> torch.Tensor:
        if self.layer_prefix_plain or self.cfg.compress_ratios[layer] == 0:
            return self.inv_plain
        return self.inv_long

    def _plane_rows(self, m: int) -> int:
        """Rows of split-K plane storage a projection with `m` outputs can need: max over pass sizes of splits x rows."""
        best = 0
        for r in range(1, self.max_rows + 1):
            bn = G.pick_bn(r)
            best = max(best, r * G.pick_splits(m, 1 << 20, max_splits=self.max_splits, n_tiles=(r + bn - 1) // bn))
        return best

    def _wo_a_splits(self, rows: int) -> int:
        """Split-K factor of the grouped wo_a projection (one batch entry per local head group)."""
        if rows > self.fused_rows:
            return 1
        kg = self.cfg.heads_per_group * self.cfg.head_dim
        return G.pick_splits(self.cfg.o_lora, kg, max_splits=self.max_splits, batch=self.GL)

    def _attn_splits(self, rows: int) -> int:
        """Key-tile splits per row: one tile per CTA for a few rows (decode), fewer and longer CTAs once the rows
        alone fill the GPU about two to three CTAs deep (prefill; one split lets the kernel write final rows)."""
        if A.tc_usable(self.cfg.head_dim, self.HL, rows, self.cache.row_bytes > 0):
            want = -(-2 * 148 // rows)           # one CTA covers every head of a row
        else:
            want = -(-3 * 148 // (rows * ((self.HL + 15) // 16)))
        return max(1, min(self.n_splits_attn, want))

    def _splits(self, m: int, k: int, rows: int) -> int:
        """Split-K factor of a swap-AB projection: fill one wave of CTAs, counting the row tiles of long passes."""
        n_tiles = (rows + G.pick_bn(rows) - 1) // G.pick_bn(rows)
        return G.pick_splits(m, k, max_splits=self.max_splits, n_tiles=n_tiles)

    def _run(self, tag, fn, *args, **kw):
        """Launch one kernel; `self.only` (a set of tags) restricts a pass to some kernels for profiling."""
        if self.only is not None and tag not in self.only:
            return
        self.launches += 1
        if self.nvtx:
            torch.cuda.nvtx.range_push(tag)
            try:
                err = fn(*args, **kw)
            finally:
                torch.cuda.nvtx.range_pop()
            if err is not None:
                lib.check(err, tag)
            return
        if self.timeline is not None:           # eager passes only: a CUDA event pair around every launch
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            err = fn(*args, **kw)
            e1.record()
            self.timeline.append((tag, e0, e1))
        else:
            err = fn(*args, **kw)
        if err is not None:
            lib.check(err, tag)

    def set_rows(self, tokens, positions, slots, row_hi=None, row_lo=None):
        """Host -> device copy of one pass's inputs (lists or CPU tensors).  `row_lo` (one position per row) puts a
        floor under the attention windows of the pass: positions below it are not attended."""
        n = len(positions)
        self._floor_on = row_lo is not None
        if row_lo is not None:
            self.row_lo.copy_(torch.tensor(list(row_lo) + [0] * (self.max_rows - n), dtype=I32), non_blocking=True)
        assert n <= self.max_rows
        pad = self.max_rows - n
        p = torch.tensor(list(positions) + [0] * pad, dtype=I32)
        s = torch.tensor(list(slots) + [-1] * pad, dtype=I32)
        if tokens is not None:        # None: the token ids are already on the device (fed by a kernel)
            assert len(tokens) == n
            self.in_tokens.copy_(torch.tensor(list(tokens) + [0] * pad, dtype=I32), non_blocking=True)
        self.row_pos.copy_(p, non_blocking=True)
        self.row_slot.copy_(s, non_blocking=True)
        # what the host knows about the pass it just described (used by the next forward_rows only): a long pass over
        # one request lets the indexer run as a tensor-core GEMM over that request's keys
        # A decode-sized pass over one request (a speculative verification, a lone request's step) scores on the tensor
        # cores too; its launches may be replayed from a graph while the context grows, so the key count is the static
        # bound (-1) and the visible count per row is worked out on the device.
        slot_list = list(slots)
        one = n > 0 and len(set(slot_list)) == 1 and slot_list[0] >= 0
        self._pass_hint = None
        if one and n > self.moe_rows:
            self._pass_hint = (n, int(max(positions)))
        elif one and getattr(self, "idx_q", None) is not None and self.max_keys <= 32768:
            self._pass_hint = (n, -1)
        if self.row_hi is not None:
            h = torch.tensor(list(row_hi if row_hi is not None else positions) + [0] * pad, dtype=I32)
            self.row_hi.copy_(h, non_blocking=True)

    # ------------------------------------------------------------------ Engram memory layers
    def attach_engram(self, layer: int, module) -> None:
        """Give decoder layer `layer` an Engram update of the streams it receives (models/engram.py EngramLayer;
        reference: rust/crates/ds41rt-daemon/src/v41_target_pass.rs:403-442)."""
        assert 0 <= layer < self.n_layers and module.H == self.cfg.hidden
        n = self.max_rows * module.rpt
        module.reserve(self.max_rows)
        module.status = self.status        # one status word for the whole pass
        host = torch.zeros(n, module.row_bytes, dtype=torch.uint8)
        if self.device.type == "cuda":
            host = host.pin_memory()
        self._engram_layer_of[id(module)] = layer
        self.engram[layer] = (module, host, torch.ones(self.max_rows, dtype=torch.uint8, device=self.device))

    def set_engram_rows(self, layer: int, rows_q, text_mask=None) -> None:
        """Table rows of the next pass for one Engram layer: uint8 [pass rows * rows_per_token, row_bytes] (numpy or a
        CPU tensor, e.g. a gather slot), `text_mask` one flag per pass row (0 = image row, streams pass through).
        The rows are copied into the engine's pinned buffer, so the caller's buffer is free on return and a captured
        pass replays against the same host address."""
        module, host, mask = self.engram[layer]
        src = rows_q if isinstance(rows_q, torch.Tensor) else torch.from_numpy(rows_q)
        n = src.shape[0]
        assert n % module.rpt == 0 and n <= host.shape[0] and src.shape[1] == module.row_bytes
        ev = self._engram_copied.get(layer)
        if ev is not None:
            ev.synchronize()          # the previous pass's upload reads the same pinned buffer
        host[:n].copy_(src)
        m = torch.ones(self.max_rows, dtype=torch.uint8)
        if text_mask is not None:
            m[: len(text_mask)] = torch.as_tensor(text_mask, dtype=torch.uint8)
        mask.copy_(m, non_blocking=True)
        self._engram_live.add(layer)

    def clear_engram_rows(self) -> None:
        self._engram_live.clear()

    def _mix_weight(self, fn: torch.Tensor) -> torch.Tensor:
        """[64, 4H] bf16 for the mixes GEMM: rows 0-23 the bf16 rounding of `fn`, rows 24-47 the bf16 rounding of what
        that left (together about 16 mantissa bits of the fp32 matrix), the rest zero."""
        w = self._mix_w.get(fn.data_ptr())
        if w is None:
            hi = fn.to(BF16)
            w = torch.zeros(64, fn.shape[1], dtype=BF16, device=fn.device)
            w[:24] = hi
            w[24:48] = (fn - hi.float()).to(BF16)
            self._mix_w[fn.data_ptr()] = w
        return w

    def _mix_gemm(self, streams: torch.Tensor, rows: int, fn: torch.Tensor) -> None:
        """mix_planes[split][rows][64] = streams[rows, 4H] x (high | low parts of fn)^T on the tensor cores."""
        K = self.cfg.hc_mult * self.cfg.hidden
        splits = G.pick_splits(rows, K, max_splits=16)
        planes = self.mix_planes[: splits * rows * 64]
        self._run("gemm_mix", G.gemm_raw, streams.view(-1, K)[:rows], self._mix_weight(fn), planes if splits == 1 else None,
                  rows, 64, K, lda=K, ldb=K, ldo=64, out_mode=1, k_splits=splits,
                  split_workspace=planes if splits > 1 else None, bn=64, status=self.status, static_operand=2)
        self._mix_state = (splits, rows)

    def _mix_args(self, rows: int):
        """(slices of hc_partial to sum, the four projection arguments of hc_finish): the planes of the GEMM that just
        ran and the single slice the expand kernel wrote, or the dot-product kernel's slices and no planes."""
        st, self._mix_state = self._mix_state, None
        if st is None:
            return self.n_slices, (lib.ptr(None), 0, C.c_longlong(0), 0)
        assert st[1] == rows
        return 1, (lib.ptr(self.mix_planes), st[0], C.c_longlong(rows * 64), 64)

    def _mix_tc(self, rows: int) -> bool:
        """Long passes (whose routed experts take bf16 rows through the all-to-all, so nothing reads the quantised rows
        of the fused step) run the mixes projection on the tensor cores and collapse inside the expand kernel."""
        return self.mix_planes is not None and rows >= self.mix_tc_rows and rows > self.moe_rows

    def _post_mix(self, rows, part_bases, n_ranks, n_splits, split_stride, fn, sync, coef=None, collapse=None):
        """`collapse` = (pre_in, norm_w, tap) asks the tensor-core form to collapse and normalise the rows into self.xn
        in the same launch (hc_finish then only turns the projections into the next coefficients)."""
        k, st = self.k, lib.stream()
        post, comb = coef if coef is not None else (self.post, self.comb)
        wait_flags = lib.ptr(self.flag_ptrs) if (sync and self.world > 1) else lib.ptr(None)
        tc = self._mix_tc(rows)
        if tc and collapse is not None:
            extra = (lib.ptr(collapse[0]), lib.ptr(collapse[1]), lib.ptr(self.xn), lib.ptr(collapse[2]),
                     C.c_float(self.cfg.norm_eps))
        else:
            extra = (lib.ptr(None), lib.ptr(None), lib.ptr(None), lib.ptr(None), C.c_float(0.0))
        self._run("hc_post_mix", k.ds41_hc_post_mix, 
            lib.ptr(self.streams), lib.ptr(self.streams), part_bases, n_ranks, n_splits, C.c_longlong(split_stride),
            lib.ptr(post), lib.ptr(comb), lib.ptr(None if tc else fn), lib.ptr(self.hc_partial), rows, self.cfg.hidden,
            wait_flags, lib.ptr(self.epoch), lib.ptr(self.status), *extra, st)
        if tc:
            self._mix_gemm(self.streams, rows, fn)

    def _finish(self, rows, scale, base, pre_in, norm_w, next_pre, tap=None, quant=False, coef=None, collapsed=False):
        """`collapsed`: self.xn (and the tap) were written by the expand kernel already."""
        cfg = self.cfg
        post, comb = coef if coef is not None else (self.post, self.comb)
        n_slices, mix = self._mix_args(rows)
        quant = quant and not collapsed
        self._run("hc_finish", self.k.ds41_hc_finish, 
            lib.ptr(self.hc_partial), n_slices, lib.ptr(scale), lib.ptr(base), lib.ptr(pre_in),
            lib.ptr(self.streams), lib.ptr(norm_w), lib.ptr(next_pre), lib.ptr(post), lib.ptr(comb),
            lib.ptr(None if collapsed else self.xn), lib.ptr(None if collapsed else tap),
            lib.ptr(self.xq if quant else None), lib.ptr(self.xq_sf if quant else None), rows, cfg.hidden,
            cfg.hc_sinkhorn_iters, C.c_float(cfg.hc_eps), C.c_float(cfg.norm_eps), *mix, lib.stream())

    def _step(self, rows, part_bases, n_ranks, n_splits, split_stride, coef_in, pre_in, fn, scale, base, norm_w,
              next_pre, coef_out, tap=None, quant=False, sync=False):
        cfg = self.cfg
        a = lib.HcStepArgs()
        a.streams_in = a.streams_out = lib.ptr(self.streams)
        a.part_bases = C.cast(part_bases, C.c_void_p) if part_bases is not None else None
        a.post, a.comb = lib.ptr(coef_in[0]), lib.ptr(coef_in[1])
        a.pre_in, a.fn, a.scale, a.base, a.norm_w = (lib.ptr(pre_in), lib.ptr(fn), lib.ptr(scale), lib.ptr(base),
                                                     lib.ptr(norm_w))
        a.partial, a.xc = lib.ptr(self.step_partial), lib.ptr(self.xc)
        a.next_pre, a.post_out, a.comb_out = lib.ptr(next_pre), lib.ptr(coef_out[0]), lib.ptr(coef_out[1])
        a.xn, a.tap_mean = lib.ptr(self.xn), lib.ptr(tap)
        a.xq, a.xq_sf = lib.ptr(self.xq if quant else None), lib.ptr(self.xq_sf if quant else None)
        a.tickets = lib.ptr(self.tickets)
        a.wait_flags = lib.ptr(self.flag_ptrs) if (sync and self.world > 1) else None
        a.wait_epoch, a.status = lib.ptr(self.epoch), lib.ptr(self.status)
        a.split_stride, a.n_ranks, a.n_splits = split_stride, n_ranks, n_splits
        a.rows, a.H, a.iters, a.hc_eps, a.norm_eps = rows, cfg.hidden, cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.norm_eps
        self._run("hc_step", self.k.ds41_hc_step, C.byref(a), lib.stream())

    def _signal(self):
        if self.world > 1:
            self._run("signal", self.k.ds41_signal_all, lib.ptr(self.epoch), lib.ptr(self.flag_out), self.world,
                      lib.stream())

    # ------------------------------------------------------------------ one pass over `rows` rows
    def _hc(self, rows, pending, fn, scale, base, norm_w, tap=None, quant=False, engram=None):
        """Close the pending sublayer (expand with its partial planes) and open the next one
        (mixes -> collapse -> RMSNorm into self.xn).  One fused launch for small passes, two otherwise.
        With `engram` (a layer that receives an Engram update) the step is split: expand, gated update of the
        streams, mixes recomputed on the updated streams, then collapse + norm."""
        cur = self._cur
        bases, n_ranks, n_splits, stride = pending if pending is not None else (None, 0, 0, 0)
        if engram is not None:
            module, host, mask = engram
            small = rows <= self.fused_rows
            cin = self.coef[self._ccur] if small else None
            cout = self.coef[self._ccur ^ 1] if small else None
            if pending is not None:
                self._post_mix(rows, bases, n_ranks, n_splits, stride, fn, sync=True, coef=cin)
            self._run("engram", module.apply, self.streams[:rows], host, mask)
            if self.device.type == "cuda" and not torch.cuda.is_current_stream_capturing():
                ev = torch.cuda.Event()
                ev.record()
                self._engram_copied[self._engram_layer_of[id(module)]] = ev
            fuse = self._mix_tc(rows)
            self._post_mix(rows, None, 0, 0, 0, fn, sync=False, coef=cin,
                           collapse=(self.pre[cur], norm_w, tap) if fuse else None)
            self._finish(rows, scale, base, self.pre[cur], norm_w, self.pre[cur ^ 1], tap, quant, coef=cout,
                         collapsed=fuse)
            if small:
                self._ccur ^= 1
        elif rows <= self.fused_rows:
            cc = self._ccur
            self._step(rows, bases, n_ranks, n_splits, stride, self.coef[cc], self.pre[cur], fn, scale, base, norm_w,
                       self.pre[cur ^ 1], self.coef[cc ^ 1], tap=tap, quant=quant, sync=pending is not None)
            self._ccur = cc ^ 1
        else:
            fuse = self._mix_tc(rows)
            self._post_mix(rows, bases, n_ranks, n_splits, stride, fn, sync=pending is not None,
                           collapse=(self.pre[cur], norm_w, tap) if fuse else None)
            self._finish(rows, scale, base, self.pre[cur], norm_w, self.pre[cur ^ 1], tap, quant, collapsed=fuse)
        self._cur = cur ^ 1

    def _qkv(self, l: int, lw: LayerWeights, R: int, inv, sources: bool = True):
        """Fused q_a / kv / extras projection of layer `l` from self.xn, its post-processing (norms, RoPE, window-ring
        rows) and, for a layer that produces a compressed source, the compressor (skipped with sources=False)."""
        cfg, k, st = self.cfg, self.k, lib.stream
        H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
        ntot = lw.w_qkv.shape[0]
        s_qkv = self._splits(ntot, H, R)
        self._run("gemm_qkv", G.linear_planes, self.xn[:R], lw.w_qkv,
                  self.planes_qkv.view(-1)[: s_qkv * R * ntot].view(s_qkv, R, ntot), s_qkv, status=self.status)
        self._run("qkv_post", k.ds41_qkv_post,
            lib.ptr(self.planes_qkv), s_qkv, R, ntot, Q, D, cfg.rope_dim, lw.extra_cols, lw.index_heads_cols,
            C.c_float(cfg.index_weight_scale), lib.ptr(lw.q_norm), lib.ptr(lw.kv_norm), lib.ptr(inv),
            lib.ptr(self.row_pos), lib.ptr(self.row_slot), lib.ptr(self.q_lat), lib.ptr(self.cache.win[l]),
            self.cache.ring, lib.ptr(self.extras), C.c_float(cfg.norm_eps), self.cache.row_bytes, st())
        if lw.ratio and sources:
            self._run("compress", k.ds41_compress,
                lib.ptr(self.extras), lw.extra_cols, R, D, cfg.index_dim, cfg.rope_dim, lw.ratio,
                lib.ptr(self.row_pos), lib.ptr(self.row_slot), lib.ptr(self.cache.pending.get(l)),
                lib.ptr(lw.comp_norm), lib.ptr(lw.wk_idx), lib.ptr(lw.k_norm), lib.ptr(inv), lib.ptr(self.inv_idx),
                lib.ptr(self.cache.page_table), self.cache.max_pages, self.cache.page_rows[l],
                lib.ptr(self.cache.comp[l]), lib.ptr(self.cache.idx[l]), C.c_float(cfg.norm_eps),
                -self.cache.comp_row_bytes if self.cache.comp_row_bytes else self.cache.row_bytes,
                self.cache.idx_row_bytes, st())

    def forward_rows(self, rows: int, *, embed: bool = True, head: bool = True, first_layer: int = 0,
                     last_layer: Optional[int] = None, sources: bool = True, pending=None,
                     head_row: Optional[int] = None):
        """One pass over `rows` rows described by set_rows().  `first_layer` / `last_layer` run a slice of the stack
        (the streams and the pending sublayer carry over between slices); `sources=False` leaves the compressed
        sources untouched (decoder replay of a prompt's tail)."""
        cfg, k, st = self.cfg, self.k, lib.stream
        H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
        R = rows
        last_layer = self.n_layers if last_layer is None else last_layer
        if first_layer == 0:
            self._cand_ratio = None
        if pending is None and self.sp_ready(R) and (embed or self._sp_active is not None):
            return self._forward_rows_sp(R, embed=embed, head=head, first_layer=first_layer, last_layer=last_layer,
                                         sources=sources, head_row=head_row)
        assert self._sp_active is None or embed, "a row-sharded pass cannot continue replicated"
        self._sp_active = None
        if embed:
            self._cur, self._ccur = 0, 0
            self._run("embed", k.ds41_embed_streams, lib.ptr(self.in_tokens), lib.ptr(self.w.embed), lib.ptr(self.streams),
                                          lib.ptr(self.pre[0]), R, H, cfg.hc_mult, cfg.vocab, st())
            if self.image_patch is not None:
                # rows of this pass that stand for image placeholders take the vision tower's output instead of the
                # placeholder token's embedding: (image_rows [n, H] bf16, row_ids [n] int32, -1 = not in this pass)
                img_rows, img_ids = self.image_patch
                self._run("image_rows", k.ds41_vis_scatter, lib.ptr(img_rows), lib.ptr(img_ids), lib.ptr(self.streams),
                          img_rows.shape[0], H, cfg.hc_mult, st())
        # `pending`: an unmerged sublayer handed in by the caller (bases, ranks, splits, stride), e.g. a pipeline stage
        # that continues another stage's stack
        fused = R <= self.fused_rows
        if self.layer_timer is not None:
            self.layer_timer.begin()
        for l in range(first_layer, last_layer):
            lw = self.w.layers[l]
            inv = self._inv(l)
            # ---------------- attention sublayer
            tap = None
            if self.taps is not None and cfg.dspark is not None and not self.layer_prefix_plain \
                    and l in cfg.dspark.tap_layers:
                tap_i = cfg.dspark.tap_layers.index(l)
                tap = self.taps[tap_i] if tap_i < self.taps.shape[0] else None
            self._hc(R, pending, lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, lw.attn_norm, tap=tap,
                     engram=self.engram[l] if l in self._engram_live else None)
            self._qkv(l, lw, R, inv, sources)
            src = None if self.layer_prefix_plain else cfg.source_of(l)
            nqb = lw.w_qb.shape[0]
            self._run("gemm_qb", G.gemm_raw, lw.w_qb, self.q_lat, self.qb_out, nqb, R, Q, lda=Q, ldb=Q, ldo=self.nqb, out_mode=2,
                       status=self.status, static_operand=1)
            if lw.index_heads_cols and src is not None:
                ratio = cfg.source_layers[src]
                # index layers above the candidate layer score and select only inside its candidate blocks
                restrict = self.cand_on and l > cfg.candidate_layer and self._cand_ratio == ratio
                cand = (lib.ptr(self.cand_mask), self.cand_words, cfg.candidate_block) if restrict \
                    else (lib.ptr(None), 0, 0)
                hint = self._pass_hint
                n_keys = 0
                if hint is not None and hint[0] == R:
                    # static bound: every key row the slot's page table can address (rows of pages that are not
                    # leased read as zeros and lie beyond every row's visible count)
                    n_keys = min((self.max_keys + ratio - 1) // ratio, self.cache.max_pages * self.cache.page_rows[src],
                                 self.max_keys) if hint[1] < 0 else min((hint[1] + 1) // ratio, self.max_keys)
                if n_keys >= 64 and cfg.index_heads == 32 and cfg.index_dim % 64 == 0:
                    self._run("index_prepare", k.ds41_index_prepare, lib.ptr(self.qb_out), C.c_longlong(self.nqb),
                              self.HL * D, lib.ptr(self.cache.idx[src]), lib.ptr(self.cache.page_table),
                              self.cache.max_pages, self.cache.page_rows[src], lib.ptr(self.row_pos),
                              lib.ptr(self.row_slot), lib.ptr(self.inv_idx), R, cfg.index_heads, cfg.index_dim, ratio,
                              n_keys, self.max_keys, lib.ptr(self.idx_q), lib.ptr(self.idx_k), lib.ptr(self.idx_vis),
                              self.cache.idx_row_bytes, st())
                    w_off = lw.extra_cols - cfg.index_heads
                    self._run("index_score_gemm", G.gemm_raw, self.idx_q, self.idx_k, self.scores, R * cfg.index_heads,
                              n_keys, cfg.index_dim, lda=cfg.index_dim, ldb=cfg.index_dim, ldo=self.max_keys, out_mode=8,
                              bn=256 if n_keys >= 256 else 64, row_w=self.extras[:, w_off:], row_w_ld=lw.extra_cols,
                              col_limit=self.idx_vis, status=self.status)
                else:
                    self._run("index_score", k.ds41_index_score_cand,
                        lib.ptr(self.qb_out), C.c_longlong(self.nqb), self.HL * D, lib.ptr(self.extras), lw.extra_cols,
                        lw.extra_cols - cfg.index_heads, lib.ptr(self.cache.idx[src]), lib.ptr(self.cache.page_table),
                        self.cache.max_pages, self.cache.page_rows[src], lib.ptr(self.row_pos), lib.ptr(self.row_slot),
                        lib.ptr(self.inv_idx), R, cfg.index_heads, cfg.index_dim, ratio, lib.ptr(self.scores),
                        self.max_keys, *cand, self.cache.idx_row_bytes, st())
                if self.cand_on and l == cfg.candidate_layer:
                    self._run("candidate_select", k.ds41_candidate_select, lib.ptr(self.scores), self.max_keys,
                              lib.ptr(self.row_pos), lib.ptr(self.row_slot), ratio, cfg.candidate_block,
                              cfg.candidate_topk_blocks, lib.ptr(self.cand_blocks), lib.ptr(self.cand_count),
                              lib.ptr(self.cand_mask), self.cand_words, R, st())
                    self._cand_ratio = ratio
                self._run("topk", k.ds41_topk_select_cand, lib.ptr(self.scores), self.max_keys, lib.ptr(self.row_pos),
                                            lib.ptr(self.row_slot), ratio, cfg.index_topk, lib.ptr(self.sel),
                                            lib.ptr(self.n_sel), R, *cand, st())
            self._run("attend", A.attend, q=self.qb_out, ldq=self.nqb, q_off=0, rows=R, heads=self.HL, D=D,
                      window=cfg.window, ring=self.cache.ring, row_pos=self.row_pos, row_slot=self.row_slot,
                      win=self.cache.win[l], comp_pool=self.cache.comp[src] if src is not None else None,
                      sel=self.sel, n_sel=self.n_sel, k=cfg.index_topk, page_table=self.cache.page_table,
                      max_pages=self.cache.max_pages, page_rows=self.cache.page_rows[src] if src is not None else 1,
                      inv_freq=inv, rope_dim=cfg.rope_dim, scale=cfg.softmax_scale, n_splits=self._attn_splits(R),
                      part_o=self.part_o, part_ml=self.part_ml, sink=lw.sink, out=self.attn_out, ldo=self.HL * D,
                      kv_row_bytes=self.cache.row_bytes, comp_row_bytes=self.cache.comp_row_bytes,
                      row_hi=self.row_hi, row_lo=self.row_lo if self._floor_on else None, status=self.status)
            # grouped wo_a: batch = local groups
            kg = cfg.heads_per_group * D
            s_a = self._wo_a_splits(R)
            if s_a > 1:
                # few rows: the K loop of one CTA per (group, 128 outputs) is a latency chain, so it is split over
                # CTAs and the fp32 partials are summed into the bf16 rows by one small kernel
                self._run("gemm_wo_a", G.gemm_raw, lw.wo_a, self.attn_out, None, cfg.o_lora, R, kg, lda=kg,
                          ldb=self.HL * D, ldo=cfg.o_lora, out_mode=3, k_splits=s_a, split_workspace=self.planes_oa,
                          batch=self.GL, a_batch_stride=cfg.o_lora * kg, b_batch_stride=kg, status=self.status,
                          static_operand=1)
                self._run("reduce_groups", k.ds41_reduce_groups, lib.ptr(self.planes_oa), s_a, self.GL, R, cfg.o_lora,
                          lib.ptr(self.oa), C.c_longlong(self.GL * cfg.o_lora), st())
            else:
                self._run("gemm_wo_a", G.gemm_raw, lw.wo_a, self.attn_out, self.oa, cfg.o_lora, R, kg, lda=kg,
                          ldb=self.HL * D, ldo=self.GL * cfg.o_lora, out_mode=2, batch=self.GL,
                          a_batch_stride=cfg.o_lora * kg, b_batch_stride=kg, out_batch_stride=cfg.o_lora,
                          status=self.status, static_operand=1)
            ko = self.GL * cfg.o_lora
            s_o = self._splits(H, ko, R)
            # the CTA of wo_b that finishes last publishes "this rank's attention planes are complete"
            self._run("gemm_wo_b", G.linear_planes, self.oa[:R], lw.wo_b, self.planes_o.view(-1)[: s_o * R * H].view(s_o, R, H), s_o,
                            status=self.status, signal=self._sig_attn)
            pending = (self._o_bases, self.world, s_o, R * H)
            # ---------------- MoE sublayer
            self._hc(R, pending, lw.hc_ffn_fn, lw.hc_ffn_scale, lw.hc_ffn_base, lw.ffn_norm, quant=self.mx)
            ng = lw.w_gate_sh.shape[0]
            s_g = self._splits(ng, H, R)
            self._run("gemm_gate", G.linear_planes, self.xn[:R], lw.w_gate_sh, self.planes_gate.view(-1)[: s_g * R * ng].view(s_g, R, ng),
                            s_g, status=self.status)
            self._run("router_select", k.ds41_router_select, 
                lib.ptr(self.planes_gate), s_g, R, ng, lw.n_experts, self.I_sh, lw.topk, lib.ptr(lw.gate_bias),
                C.c_float(cfg.route_scale), C.c_float(cfg.swiglu_limit), lib.ptr(self.ids), lib.ptr(self.route_w),
                lib.ptr(self.shared_act), st())
            if self.debug is not None:
                self.debug.append({"layer": l, "ids": self.ids[:R].clone(), "sel": self.sel[:R].clone(),
                                   "n_sel": self.n_sel[:R].clone()})
            folded = False           # did the sublayer's last kernel publish the plane itself?
            if R > self.moe_rows:
                self._moe_sorted(R, lw)
            else:
                EL = lw.n_experts // self.world
                self._run("moe_plan", k.ds41_moe_plan, 
                    lib.ptr(self.ids), lib.ptr(self.route_w), lib.ptr(self.row_slot), R, lw.topk, self.rank * EL,
                    (self.rank + 1) * EL, self.max_active, self.moe_rows, lib.ptr(self.active), lib.ptr(self.n_active),
                    lib.ptr(self.row_w), lib.ptr(self.slot_of), st())
                I = cfg.inter
                bn = G.pick_bn(R)
                # FC1: act[slot][row][i] = swiglu(W1 x, W3 x) * route weight;  FC2: fc2[slot][row][h]
                if self.nv:
                    ra = (R + 127) // 128
                    zero = C.c_longlong(0)
                    self._run("act_quant x", k.ds41_act_quant_nvfp4_rows, lib.ptr(self.xn), C.c_longlong(H),
                              lib.ptr(self.xq4), C.c_longlong(H), lib.ptr(self.xq4_sf), R, H,
                              C.c_float(NVFP4_IN_SCALE_FC1), None, 1, zero, zero, zero, None, st())
                    self._run("gemm_fc1", G.gemm_raw, lw.w13, self.xq4, self.act, I, R, H, lda=H, ldb=H, ldo=I, kind=3,
                              out_mode=4, bn=max(bn, 32), batch=self.max_active, a_batches=EL, a_batch_stride=2 * I * H,
                              out_batch_stride=R * I, batch_map=self.active, n_active=self.n_active, b_batch_kind=1,
                              up_row_offset=I, row_w=self.row_w, row_w_ld=self.moe_rows, act_limit=cfg.swiglu_limit,
                              sfa=lw.w13_sf, sfa_batch_stride=lw.w13_sf[0].numel(), sfb=self.xq4_sf, status=self.status,
                              alpha=NVFP4_IN_SCALE_FC1, alpha_batch=lw.w13_gs)
                    sf_slot = ra * (I // 64) * 512
                    self._run("act_quant act", k.ds41_act_quant_nvfp4_rows, lib.ptr(self.act), C.c_longlong(I),
                              lib.ptr(self.actq4), C.c_longlong(I), lib.ptr(self.actq4_sf), R, I,
                              C.c_float(NVFP4_IN_SCALE_FC2), None, self.max_active, C.c_longlong(R * I),
                              C.c_longlong(R * I), C.c_longlong(sf_slot), lib.ptr(self.n_active), st())
                    self._run("gemm_fc2", G.gemm_raw, lw.w2, self.actq4, self.fc2, H, R, I, lda=I, ldb=I, ldo=H, kind=3,
                              out_mode=5, bn=max(bn, 32), batch=self.max_active, a_batches=EL, a_batch_stride=H * I,
                              b_batch_stride=R * I, out_batch_stride=R * H, batch_map=self.active,
                              n_active=self.n_active, b_batch_kind=2, row_w=self.row_w, row_w_ld=self.moe_rows,
                              sfa=lw.w2_sf, sfa_batch_stride=lw.w2_sf[0].numel(), sfb=self.actq4_sf,
                              sfb_batch_stride=sf_slot, status=self.status, alpha=NVFP4_IN_SCALE_FC2,
                              alpha_batch=lw.w2_gs)
                elif self.mx:
                    ra = (R + 127) // 128
                    self._run("gemm_fc1", G.gemm_raw, lw.w13, self.xq, self.act, I, R, H, lda=H, ldb=H, ldo=I, kind=2, out_mode=4, bn=bn,
                               batch=self.max_active, a_batches=EL, a_batch_stride=2 * I * H, out_batch_stride=R * I,
                               batch_map=self.active, n_active=self.n_active, b_batch_kind=1, up_row_offset=I,
                               row_w=self.row_w, row_w_ld=self.moe_rows, act_limit=cfg.swiglu_limit,
                               sfa=lw.w13_sf, sfa_batch_stride=lw.w13_sf[0].numel(), sfb=self.xq_sf, status=self.status,
                               a_format=self.a_fmt)
                    sf_slot = ra * (I // 128) * 512
                    self._run("act_quant act", k.ds41_act_quant_mx, lib.ptr(self.act), C.c_longlong(I), C.c_longlong(R * I),
                                                 lib.ptr(self.actq), C.c_longlong(I), C.c_longlong(R * I),
                                                 lib.ptr(self.actq_sf), C.c_longlong(sf_slot), R, I, self.max_active, 128,
                                                 lib.ptr(self.n_active), st())
                    self._run("gemm_fc2", G.gemm_raw, lw.w2, self.actq, self.fc2, H, R, I, lda=I, ldb=I, ldo=H, kind=2, out_mode=5, bn=bn,
                               batch=self.max_active, a_batches=EL, a_batch_stride=H * I, b_batch_stride=R * I,
                               out_batch_stride=R * H, batch_map=self.active, n_active=self.n_active, b_batch_kind=2,
                               row_w=self.row_w, row_w_ld=self.moe_rows, sfa=lw.w2_sf,
                               sfa_batch_stride=lw.w2_sf[0].numel(), sfb=self.actq_sf, sfb_batch_stride=sf_slot,
                               status=self.status, a_format=self.a_fmt)
                else:
                    self._run("gemm_fc1", G.gemm_raw, lw.w13, self.xn, self.act, I, R, H, lda=H, ldb=H, ldo=I, out_mode=4, bn=bn,
                               batch=self.max_active, a_batches=EL, a_batch_stride=2 * I * H, out_batch_stride=R * I,
                               batch_map=self.active, n_active=self.n_active, b_batch_kind=1, up_row_offset=I,
                               row_w=self.row_w, row_w_ld=self.moe_rows, act_limit=cfg.swiglu_limit, status=self.status)
                    self._run("gemm_fc2", G.gemm_raw, lw.w2, self.act, self.fc2, H, R, I, lda=I, ldb=I, ldo=H, out_mode=5, bn=bn,
                               batch=self.max_active, a_batches=EL, a_batch_stride=H * I, b_batch_stride=R * I,
                               out_batch_stride=R * H, batch_map=self.active, n_active=self.n_active, b_batch_kind=2,
                               row_w=self.row_w, row_w_ld=self.moe_rows, status=self.status)
                s_s = self._splits(H, self.I_sh, R)
                self._run("gemm_shared_down", G.linear_planes, self.shared_act[:R], lw.w2_sh,
                                self.planes_shared.view(-1)[: s_s * R * H].view(s_s, R, H), s_s, status=self.status)
                if self.world > 1:       # the block that finishes last publishes the expert plane
                    self._run("moe_combine", k.ds41_moe_combine_signal, lib.ptr(self.fc2), lib.ptr(self.slot_of),
                              lib.ptr(self.planes_shared), s_s, R, lw.topk, H, lib.ptr(self.moe_plane),
                              lib.ptr(self.sig_counters[1:2]), lib.ptr(self.epoch), lib.ptr(self.flag_out), self.world, st())
                else:
                    self._run("moe_combine", k.ds41_moe_combine, lib.ptr(self.fc2), lib.ptr(self.slot_of), lib.ptr(self.planes_shared), s_s,
                                                R, lw.topk, H, lib.ptr(self.moe_plane), st())
                folded = True
            if not folded:
                self._signal()
            pending = (self._moe_bases, self.world, 1, 0)
            if self.layer_timer is not None:
                self.layer_timer.mark()
            if self.activation_trace is not None:
                # the layer's output is merged into the streams by the next sublayer; the dump shows the streams as
                # they stand plus the pending expert plane of this rank
                self.activation_trace.dump(l, self.streams, self.row_pos, R)
        self._pending = pending
        if self._pass_hint is not None and self._pass_hint[1] >= 0:
            self._pass_hint = None        # a long pass's key count holds for that pass only; the static form stays until
                                          # the rows are described again (device-fed steps keep their slot)
        if head:
            self.head_rows(R if head_row is None else head_row + 1)


    # ------------------------------------------------------------------ sequence-parallel long passes
    def sp_ready(self, rows: int) -> bool:
        """Can a pass of `rows` rows run row-sharded (see `long_pass` in the constructor)?"""
        if self.long_pass == "replicated" or rows <= self.moe_rows or self._engram_live:
            return False
        if self.world == 1 and self.long_pass != "sp":
            return False
        lw = self._lw_any
        return rows % (128 * self.world) == 0 and lw is not None and lw.w_qb_full is not None \
            and self.cfg.n_heads <= 64

    def sp_rows(self, n: int) -> int:
        """Rows to run for a chunk of n real rows: padded up to the row-sharded granularity when that fits."""
        g = 128 * self.world
        padded = (n + g - 1) // g * g
        return padded if padded <= self.max_rows and self.sp_ready(padded) else n

    def _sp_buffers(self, Rl: int):
        cfg, dev = self.cfg, self.device
        if self._sp is not None and self._sp["Rl"] >= Rl:
            return self._sp
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
        D, NH = cfg.head_dim, cfg.n_heads
        nqb = NH * D + cfg.index_heads * cfg.index_dim
        splits = max(1, min(self.n_splits_attn, -(-2 * 148 // Rl)))
        ng = self.E + 2 * cfg.inter
        self._sp = dict(
            Rl=Rl, nqb=nqb, qb=z((Rl, nqb), BF16), attn=z((Rl, NH * D), BF16), oa=z((Rl, cfg.o_groups * cfg.o_lora), BF16),
            # the tensor-core kernel writes final rows when it has one split; the warp-MMA kernels always go through
            # partials
            part_o=z((Rl * splits if splits > 1 or not A.tc_usable(D, NH, Rl, self.cache.row_bytes > 0) else 1, NH, D), F32),
            part_ml=z((Rl * splits, NH, 2), F32),
            planes_o=z((self.max_splits * Rl * cfg.hidden,), F32), planes_gate=z((self.max_splits * Rl * ng,), F32),
            shared_act=z((Rl, cfg.inter), BF16), planes_shared=z((self.max_splits * Rl * cfg.hidden,), F32),
            xn_last=z((1, cfg.hidden), BF16))
        return self._sp

    def _sp_gather_ctx(self, Rl: int):
        """Symmetric buffers of the fused all-gather -> GEMM for `Rl` rows per rank: two alternating copies of the
        gathered [world * Rl, H] matrix, arrival counters per (source, 128-row tile) and a private call counter."""
        ctx = self._sp_ag.get(Rl)
        if ctx is None:
            from ..parallel.tp import SyncFlags
            W, H = self.world, self.cfg.hidden
            full = W * Rl * H * 2
            x_sym = self.fabric.alloc(2 * full)
            ctx = dict(x_sym=x_sym, full=full, parity=0, calls=SyncFlags(self.fabric),
                       arrive=self.fabric.alloc(4 * W * (Rl // 128)),
                       views=[x_sym.view(BF16, (W * Rl, H), i * full) for i in range(2)])
            self._sp_ag[Rl] = ctx
        return ctx

    def _sp_hc(self, lo, Rl, pending, fn, scale, base, norm_w, xn_out, tap=None):
        """Own rows [lo, lo + Rl): close the pending sublayer (its planes are local and complete) and open the next
        one; the normalised rows go to `xn_out` ([Rl, H] bf16)."""
        cfg, cur = self.cfg, self._cur
        bases, n_splits, stride = pending if pending is not None else (None, 0, 0)
        ptrs = (C.c_void_p * 1)(bases) if bases is not None else None
        streams = self.streams[lo:]
        tc = self._mix_tc(Rl)
        tap_lo = tap[lo:] if tap is not None else None
        extra = (lib.ptr(self.pre[cur][lo:]), lib.ptr(norm_w), lib.ptr(xn_out), lib.ptr(tap_lo),
                 C.c_float(cfg.norm_eps)) if tc else \
            (lib.ptr(None), lib.ptr(None), lib.ptr(None), lib.ptr(None), C.c_float(0.0))
        self._run("hc_post_mix", self.k.ds41_hc_post_mix, lib.ptr(streams), lib.ptr(streams), ptrs,
                  1 if bases is not None else 0, n_splits, C.c_longlong(stride), lib.ptr(self.post[lo:]),
                  lib.ptr(self.comb[lo:]), lib.ptr(None if tc else fn), lib.ptr(self.hc_partial), Rl, cfg.hidden,
                  lib.ptr(None), lib.ptr(self.epoch), lib.ptr(self.status), *extra, lib.stream())
        if tc:
            self._mix_gemm(streams, Rl, fn)
        n_slices, mix = self._mix_args(Rl)
        self._run("hc_finish", self.k.ds41_hc_finish, lib.ptr(self.hc_partial), n_slices, lib.ptr(scale),
                  lib.ptr(base), lib.ptr(self.pre[cur][lo:]), lib.ptr(streams), lib.ptr(norm_w),
                  lib.ptr(self.pre[cur ^ 1][lo:]), lib.ptr(self.post[lo:]), lib.ptr(self.comb[lo:]),
                  lib.ptr(None if tc else xn_out), lib.ptr(None if tc else tap_lo), lib.ptr(None), lib.ptr(None), Rl,
                  cfg.hidden, cfg.hc_sinkhorn_iters, C.c_float(cfg.hc_eps), C.c_float(cfg.norm_eps), *mix, lib.stream())
        self._cur = cur ^ 1

    def _sp_qkv(self, l, lw, R, Rl, inv, sources, ctx):
        """q_a / kv / extras of every row on every rank: the own normalised rows (already written into the gathered
        matrix) are pushed to the peers inside the GEMM kernel, which multiplies remote row tiles as they arrive."""
        cfg, k, W = self.cfg, self.k, self.world
        H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
        ntot = lw.w_qkv.shape[0]
        planes = self.planes_qkv.view(-1)[: R * ntot].view(R, ntot)
        xfull = ctx["views"][ctx["parity"]]
        if W == 1:
            self._run("gemm_qkv", G.gemm_raw, xfull, lw.w_qkv, planes, R, ntot, H, lda=H, ldb=H, ldo=ntot, out_mode=1,
                      bn=256, status=self.status, static_operand=2)
        else:
            ctx["calls"].signal()
            a = lib.GemmArgs()
            a.B, a.out, a.status = lib.ptr(lw.w_qkv), lib.ptr(planes), lib.ptr(self.status)
            a.lda, a.ldb, a.ldo = H, lw.w_qkv.stride(0), ntot
            a.M, a.N, a.K, a.batch = R, ntot, H, 1
            a.kind, a.out_mode, a.k_splits, a.bn = 0, 1, 1, 256
            a.static_operand = 2
            a.ag_world, a.ag_rank, a.ag_rows = W, self.rank, Rl
            for r in range(W):
                a.a_peers[r] = ctx["x_sym"].peer_ptrs[r] + ctx["parity"] * ctx["full"]
                a.ag_arrive[r] = ctx["arrive"].peer_ptrs[r]
            a.ag_epoch = lib.ptr(ctx["calls"].epoch)
            self._run("gemm_qkv", lambda: lib.kernels().ds41_gemm_tc(C.byref(a), lib.stream()))
        ctx["parity"] ^= 1
        self._run("qkv_post", k.ds41_qkv_post, lib.ptr(planes), 1, R, ntot, Q, D, cfg.rope_dim, lw.extra_cols,
                  lw.index_heads_cols, C.c_float(cfg.index_weight_scale), lib.ptr(lw.q_norm), lib.ptr(lw.kv_norm),
                  lib.ptr(inv), lib.ptr(self.row_pos), lib.ptr(self.row_slot), lib.ptr(self.q_lat),
                  lib.ptr(self.cache.win[l]), self.cache.ring, lib.ptr(self.extras), C.c_float(cfg.norm_eps),
                  self.cache.row_bytes, lib.stream())
        if lw.ratio and sources:
            self._run("compress", k.ds41_compress, lib.ptr(self.extras), lw.extra_cols, R, D, cfg.index_dim,
                      cfg.rope_dim, lw.ratio, lib.ptr(self.row_pos), lib.ptr(self.row_slot),
                      lib.ptr(self.cache.pending.get(l)), lib.ptr(lw.comp_norm), lib.ptr(lw.wk_idx), lib.ptr(lw.k_norm),
                      lib.ptr(inv), lib.ptr(self.inv_idx), lib.ptr(self.cache.page_table), self.cache.max_pages,
                      self.cache.page_rows[l], lib.ptr(self.cache.comp[l]), lib.ptr(self.cache.idx[l]),
                      C.c_float(cfg.norm_eps),
                      -self.cache.comp_row_bytes if self.cache.comp_row_bytes else self.cache.row_bytes,
                      self.cache.idx_row_bytes, lib.stream())

    def _forward_rows_sp(self, R, *, embed, head, first_layer, last_layer, sources, head_row):
        cfg, k, st = self.cfg, self.k, lib.stream
        H, D, Q, W = cfg.hidden, cfg.head_dim, cfg.q_lora, self.world
        Rl = R // W
        lo = self.rank * Rl
        sp = self._sp_buffers(Rl)
        ctx = self._sp_gather_ctx(Rl)
        NH, nqb = cfg.n_heads, sp["nqb"]
        pos, slot = self.row_pos[lo:], self.row_slot[lo:]
        if embed:
            self._cur, self._ccur = 0, 0
            self._run("embed", k.ds41_embed_streams, lib.ptr(self.in_tokens), lib.ptr(self.w.embed),
                      lib.ptr(self.streams), lib.ptr(self.pre[0]), R, H, cfg.hc_mult, cfg.vocab, st())
            if self.image_patch is not None:
                img_rows, img_ids = self.image_patch
                self._run("image_rows", k.ds41_vis_scatter, lib.ptr(img_rows), lib.ptr(img_ids), lib.ptr(self.streams),
                          img_rows.shape[0], H, cfg.hc_mult, st())
            self._sp_pending = None
        self._sp_active = (lo, Rl, R)
        pending = self._sp_pending
        if self.layer_timer is not None:
            self.layer_timer.begin()
        attn_splits = max(1, min(self.n_splits_attn, -(-2 * 148 // Rl)))
        for l in range(first_layer, last_layer):
            lw = self.w.layers[l]
            inv = self._inv(l)
            tap = None
            if self.taps is not None and cfg.dspark is not None and not self.layer_prefix_plain \
                    and l in cfg.dspark.tap_layers:
                tap_i = cfg.dspark.tap_layers.index(l)
                tap = self.taps[tap_i] if tap_i < self.taps.shape[0] else None
            # ---------------- attention sublayer
            xfull = ctx["views"][ctx["parity"]]
            self._sp_hc(lo, Rl, pending, lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, lw.attn_norm, xfull[lo:],
                        tap=tap)
            self._sp_qkv(l, lw, R, Rl, inv, sources, ctx)
            src = None if self.layer_prefix_plain else cfg.source_of(l)
            nq = lw.w_qb_full.shape[0]
            self._run("gemm_qb", G.gemm_raw, lw.w_qb_full, self.q_lat[lo:], sp["qb"], nq, Rl, Q, lda=Q, ldb=Q, ldo=nqb,
                      out_mode=2, status=self.status, static_operand=1)
            if lw.index_heads_cols and src is not None:
                ratio = cfg.source_layers[src]
                restrict = self.cand_on and l > cfg.candidate_layer and self._cand_ratio == ratio
                cand = (lib.ptr(self.cand_mask[lo:]), self.cand_words, cfg.candidate_block) if restrict \
                    else (lib.ptr(None), 0, 0)
                hint = self._pass_hint        # rows beyond the hinted count are padding (slot -1: no visible key)
                n_keys = min((hint[1] + 1) // ratio, self.max_keys) if hint is not None and hint[0] <= R else 0
                scores = self.scores[lo:]
                # qkv_post packs the extras rows with this layer's own width, not the buffer's
                extras_own = self.extras.view(-1)[lo * lw.extra_cols:]
                if n_keys >= 64 and cfg.index_heads == 32 and cfg.index_dim % 64 == 0:
                    self._run("index_prepare", k.ds41_index_prepare, lib.ptr(sp["qb"]), C.c_longlong(nqb), NH * D,
                              lib.ptr(self.cache.idx[src]), lib.ptr(self.cache.page_table), self.cache.max_pages,
                              self.cache.page_rows[src], lib.ptr(pos), lib.ptr(slot), lib.ptr(self.inv_idx), Rl,
                              cfg.index_heads, cfg.index_dim, ratio, n_keys, self.max_keys, lib.ptr(self.idx_q),
                              lib.ptr(self.idx_k), lib.ptr(self.idx_vis), self.cache.idx_row_bytes, st())
                    w_off = lw.extra_cols - cfg.index_heads
                    self._run("index_score_gemm", G.gemm_raw, self.idx_q, self.idx_k, scores, Rl * cfg.index_heads,
                              n_keys, cfg.index_dim, lda=cfg.index_dim, ldb=cfg.index_dim, ldo=self.max_keys,
                              out_mode=8, bn=256 if n_keys >= 256 else 64, row_w=extras_own[w_off:],
                              row_w_ld=lw.extra_cols, col_limit=self.idx_vis, status=self.status)
                else:
                    self._run("index_score", k.ds41_index_score_cand, lib.ptr(sp["qb"]), C.c_longlong(nqb), NH * D,
                              lib.ptr(extras_own), lw.extra_cols, lw.extra_cols - cfg.index_heads,
                              lib.ptr(self.cache.idx[src]), lib.ptr(self.cache.page_table), self.cache.max_pages,
                              self.cache.page_rows[src], lib.ptr(pos), lib.ptr(slot), lib.ptr(self.inv_idx), Rl,
                              cfg.index_heads, cfg.index_dim, ratio, lib.ptr(scores), self.max_keys, *cand,
                              self.cache.idx_row_bytes, st())
                if self.cand_on and l == cfg.candidate_layer:
                    self._run("candidate_select", k.ds41_candidate_select, lib.ptr(scores), self.max_keys, lib.ptr(pos),
                              lib.ptr(slot), ratio, cfg.candidate_block, cfg.candidate_topk_blocks,
                              lib.ptr(self.cand_blocks[lo:]), lib.ptr(self.cand_count[lo:]),
                              lib.ptr(self.cand_mask[lo:]), self.cand_words, Rl, st())
                    self._cand_ratio = ratio
                self._run("topk", k.ds41_topk_select_cand, lib.ptr(scores), self.max_keys, lib.ptr(pos), lib.ptr(slot),
                          ratio, cfg.index_topk, lib.ptr(self.sel[lo:]), lib.ptr(self.n_sel[lo:]), Rl, *cand, st())
            self._run("attend", A.attend, q=sp["qb"], ldq=nqb, q_off=0, rows=Rl, heads=NH, D=D, window=cfg.window,
                      ring=self.cache.ring, row_pos=pos, row_slot=slot, win=self.cache.win[l],
                      comp_pool=self.cache.comp[src] if src is not None else None, sel=self.sel[lo:],
                      n_sel=self.n_sel[lo:], k=cfg.index_topk, page_table=self.cache.page_table,
                      max_pages=self.cache.max_pages, page_rows=self.cache.page_rows[src] if src is not None else 1,
                      inv_freq=inv, rope_dim=cfg.rope_dim, scale=cfg.softmax_scale, n_splits=attn_splits,
                      part_o=sp["part_o"], part_ml=sp["part_ml"], sink=lw.sink_full, out=sp["attn"], ldo=NH * D,
                      kv_row_bytes=self.cache.row_bytes, comp_row_bytes=self.cache.comp_row_bytes,
                      row_hi=self.row_hi[lo:] if self.row_hi is not None else None,
                      row_lo=self.row_lo[lo:] if self._floor_on else None, status=self.status)
            kg = cfg.heads_per_group * D
            ko = cfg.o_groups * cfg.o_lora
            self._run("gemm_wo_a", G.gemm_raw, lw.wo_a_full, sp["attn"], sp["oa"], cfg.o_lora, Rl, kg, lda=kg,
                      ldb=NH * D, ldo=ko, out_mode=2, batch=cfg.o_groups, a_batch_stride=cfg.o_lora * kg,
                      b_batch_stride=kg, out_batch_stride=cfg.o_lora, status=self.status, static_operand=1)
            s_o = self._splits(H, ko, Rl)
            planes_o = sp["planes_o"][: s_o * Rl * H].view(s_o, Rl, H)
            self._run("gemm_wo_b", G.linear_planes, sp["oa"][:Rl], lw.wo_b_full, planes_o, s_o, status=self.status)
            pending = (planes_o.data_ptr(), s_o, Rl * H)
            # ---------------- MoE sublayer: router and shared expert on the own rows, routed experts by all-to-all
            xn = self.xn[lo:lo + Rl]
            self._sp_hc(lo, Rl, pending, lw.hc_ffn_fn, lw.hc_ffn_scale, lw.hc_ffn_base, lw.ffn_norm, xn)
            ng = lw.w_gate_full.shape[0]
            I_all = (ng - lw.n_experts) // 2
            s_g = self._splits(ng, H, Rl)
            planes_g = sp["planes_gate"][: s_g * Rl * ng].view(s_g, Rl, ng)
            self._run("gemm_gate", G.linear_planes, xn, lw.w_gate_full, planes_g, s_g, status=self.status)
            self._run("router_select", k.ds41_router_select, lib.ptr(planes_g), s_g, Rl, ng, lw.n_experts, I_all,
                      lw.topk, lib.ptr(lw.gate_bias), C.c_float(cfg.route_scale), C.c_float(cfg.swiglu_limit),
                      lib.ptr(self.ids[lo:]), lib.ptr(self.route_w[lo:]), lib.ptr(sp["shared_act"]), st())
            if self.debug is not None:
                self.debug.append({"layer": l, "ids": self.ids[lo:lo + Rl].clone(), "sel": self.sel[lo:lo + Rl].clone(),
                                   "n_sel": self.n_sel[lo:lo + Rl].clone(), "rows": (lo, lo + Rl)})
            s_s = self._splits(H, I_all, Rl)
            planes_s = sp["planes_shared"][: s_s * Rl * H].view(s_s, Rl, H)
            self._run("gemm_shared_down", G.linear_planes, sp["shared_act"][:Rl], lw.w2_sh_full, planes_s, s_s,
                      status=self.status)
            moe_rows = self.moe_plane[lo:lo + Rl]
            self._run("reduce_planes", k.ds41_reduce_planes, lib.ptr(planes_s), s_s, C.c_longlong(Rl * H),
                      lib.ptr(moe_rows), 0, C.c_longlong(Rl * H), st())
            if self._ep is None:
                self._make_ep(lw)
            ep = self._ep
            ep.set_weights(lw.w13, lw.w2, getattr(lw, "w13_sf", None), getattr(lw, "w2_sf", None),
                           getattr(lw, "w13_gs", None), getattr(lw, "w2_gs", None))
            if self.only is None or "ep_moe" in self.only:
                self.launches += 7
                self._run("ep_moe", ep.forward, xn, self.ids[lo:lo + Rl], self.route_w[lo:lo + Rl], moe_rows, moe_rows)
            pending = (moe_rows.data_ptr(), 1, 0)
            if self.layer_timer is not None:
                self.layer_timer.mark()
            if self.activation_trace is not None:
                self.activation_trace.dump(l, self.streams, self.row_pos, R)
        self._sp_pending = pending
        self._pending = None
        self._pass_hint = None
        if head:
            self.head_rows(R if head_row is None else head_row + 1)

    def _sp_close(self, fn, scale, base, norm_w):
        """Merge the pending sublayer of a row-sharded pass and normalise: own rows of self.xn are valid afterwards."""
        lo, Rl, R = self._sp_active
        self._sp_hc(lo, Rl, self._sp_pending, fn, scale, base, norm_w, self.xn[lo:lo + Rl])
        self._sp_pending = None

    def _sp_head(self, rows: int):
        """Head of a row-sharded pass: the owner of row rows - 1 hands its normalised row to every rank (one H-wide
        broadcast), then the vocabulary shards are multiplied as usual; the logits land in row 0."""
        lo, Rl, R = self._sp_active
        lw0 = self._lw_any
        self._sp_close(lw0.hc_attn_fn, lw0.hc_attn_scale, lw0.hc_attn_base, self.w.final_norm)
        last = rows - 1
        row = self._sp["xn_last"]
        owner = last // Rl
        if owner == self.rank:
            row.copy_(self.xn[last:last + 1])
        if self.world > 1:
            import torch.distributed as dist
            dist.broadcast(row, src=owner, group=self.fabric.group)
        self._sp_active = None
        return row

    def _make_ep(self, lw: LayerWeights):
        from ..parallel.ep import ExpertParallelMoE
        per_rank = (self.max_rows + self.world - 1) // self.world
        self._ep = ExpertParallelMoE(self.fabric, lw.w13, lw.w2, topk=lw.topk, max_tokens=per_rank,
                                     act_limit=self.cfg.swiglu_limit, w13_sf=getattr(lw, "w13_sf", None),
                                     w2_sf=getattr(lw, "w2_sf", None), fp4=self.a_fmt == 1,
                                     nvfp4=(NVFP4_IN_SCALE_FC1, NVFP4_IN_SCALE_FC2) if self.nv else None,
                                     w13_gs=getattr(lw, "w13_gs", None), w2_gs=getattr(lw, "w2_gs", None))

    def _moe_sorted(self, R: int, lw: LayerWeights):
        """Routed + shared experts of a long pass: this rank's slice of the rows is dispatched to the experts' owners,
        multiplied as expert groups and combined back (parallel/ep.py); the plane every rank publishes holds its
        partial shared expert for all rows plus the complete routed sum of its own slice."""
        cfg, k, st, H = self.cfg, self.k, lib.stream, self.cfg.hidden
        s_s = self._splits(H, self.I_sh, R)
        self._run("gemm_shared_down", G.linear_planes, self.shared_act[:R], lw.w2_sh,
                  self.planes_shared.view(-1)[: s_s * R * H].view(s_s, R, H), s_s, status=self.status)
        self._run("reduce_planes", k.ds41_reduce_planes, lib.ptr(self.planes_shared), s_s, C.c_longlong(R * H),
                  lib.ptr(self.moe_plane), 0, C.c_longlong(R * H), st())
        if self._ep is None:
            self._make_ep(lw)
        lo, hi = R * self.rank // self.world, R * (self.rank + 1) // self.world
        ep = self._ep
        ep.set_weights(lw.w13, lw.w2, getattr(lw, "w13_sf", None), getattr(lw, "w2_sf", None),
                       getattr(lw, "w13_gs", None), getattr(lw, "w2_gs", None))
        if self.only is None or "ep_moe" in self.only:
            self.launches += 7
            self._run("ep_moe", ep.forward, self.xn[lo:hi], self.ids[lo:hi], self.route_w[lo:hi], self.moe_plane[lo:hi],
                      self.moe_plane[lo:hi])

    def head_rows(self, rows: int, mask: Optional[torch.Tensor] = None):
        """collapse -> final norm -> vocabulary shard GEMM -> greedy candidate (+ cross-rank merge)."""
        cfg, k, st = self.cfg, self.k, lib.stream
        lw0 = self._lw_any
        if mask is None:
            mask = self.head_mask      # [rows, ceil(vocab / 32)] int32 allow-bits applied by the selection kernel
        if self._sp_active is not None:
            xn, rows = self._sp_head(rows), 1
        else:
            self._hc(rows, getattr(self, "_pending", None), lw0.hc_attn_fn, lw0.hc_attn_scale, lw0.hc_attn_base,
                     self.w.final_norm)
            self._pending = None
            xn = self.xn
        self.last_head_row = rows - 1
        if rows > self.head_cap:
            # a long pass: only its last row continues the sequence; its logits land in row 0
            xn, rows, self.last_head_row = self.xn[rows - 1:rows], 1, 0
        self._run("gemm_head", G.gemm_raw, self.w.head, xn, self.logits, self.V_local, rows, cfg.hidden, lda=cfg.hidden, ldb=cfg.hidden,
                   ldo=self.V_local, out_mode=3, status=self.status, static_operand=1)
        self._run("argmax_rows", k.ds41_argmax_rows, 
            lib.ptr(self.logits), C.c_longlong(self.V_local), rows, self.V_local, self.rank * self.V_local,
            lib.ptr(mask), 0 if mask is None else mask.shape[-1], lib.ptr(self.best_val), lib.ptr(self.best_idx),
            lib.ptr(None), st())
        self._signal()
        wait_flags = lib.ptr(self.flag_ptrs) if self.world > 1 else lib.ptr(None)
        self._run("argmax_merge", k.ds41_argmax_merge, self._val_ptrs, self._idx_ptrs, self.world, rows, lib.ptr(self.chosen),
                                     wait_flags, lib.ptr(self.epoch), lib.ptr(self.status), st())

    def head_logits(self, rows: int):
        """collapse -> final norm -> vocabulary shard GEMM; leaves fp32 logits in self.logits (no selection)."""
        cfg = self.cfg
        lw0 = self._lw_any
        self._hc(rows, getattr(self, "_pending", None), lw0.hc_attn_fn, lw0.hc_attn_scale, lw0.hc_attn_base,
                 self.w.final_norm)
        self._pending = None
        self._run("gemm_head", G.gemm_raw, self.w.head, self.xn, self.logits, self.V_local, rows, cfg.hidden,
                  lda=cfg.hidden, ldb=cfg.hidden, ldo=self.V_local, out_mode=3, status=self.status, static_operand=1)

    def feed_rings(self, rows: int):
        """Write every layer's window-ring rows from the normalised hidden states currently in self.xn
        (rows/positions/slots as set by set_rows): the drafter's committed KV comes from the target's taps."""
        cfg, k, st = self.cfg, self.k, lib.stream
        H, D, Q = cfg.hidden, cfg.head_dim, cfg.q_lora
        for l, lw in enumerate(self.w.layers):
            ntot = lw.w_qkv.shape[0]
            s_qkv = self._splits(ntot, H, rows)
            self._run("gemm_qkv_feed", G.linear_planes, self.xn[:rows], lw.w_qkv,
                      self.planes_qkv.view(-1)[: s_qkv * rows * ntot].view(s_qkv, rows, ntot), s_qkv,
                      status=self.status)
            self._run("qkv_post_feed", k.ds41_qkv_post, lib.ptr(self.planes_qkv), s_qkv, rows, ntot, Q, D,
                      cfg.rope_dim, lw.extra_cols, lw.index_heads_cols, C.c_float(cfg.index_weight_scale),
                      lib.ptr(lw.q_norm), lib.ptr(lw.kv_norm), lib.ptr(self._inv(l)), lib.ptr(self.row_pos),
                      lib.ptr(self.row_slot), lib.ptr(self.q_lat), lib.ptr(self.cache.win[l]), self.cache.ring,
                      lib.ptr(self.extras), C.c_float(cfg.norm_eps), self.cache.row_bytes, st())

    # ------------------------------------------------------------------ convenience drivers
    def prefill(self, slot: int, tokens: List[int], start: int = 0, chunk: Optional[int] = None) -> int:
        """Run the prompt through the engine in chunks of up to max_rows rows; returns the greedy next token."""
        chunk = chunk or self.max_rows
        assert self.cache.ensure(slot, start + len(tokens) + 1)
        nxt = -1
        for c0 in range(0, len(tokens), chunk):
            part = tokens[c0:c0 + chunk]
            pos = list(range(start + c0, start + c0 + len(part)))
            self.set_rows(part, pos, [slot] * len(part))
            last = c0 + chunk >= len(tokens)
            # a chunk may run padded up to the row-sharded granularity (the padding rows have no slot)
            self.forward_rows(self.sp_rows(len(part)), head=last, head_row=len(part) - 1)
            if last:
                nxt = int(self.chosen[self.last_head_row].item())
        return nxt

    def boundary_source(self, rows: int, layer: int, sources: bool = True):
        """Finish an encoder slice at `layer`: merge the pending sublayer into the streams, normalise layer `layer`'s
        input and run only its projection + compressor, so that its compressed source covers these rows.  Afterwards
        self.streams holds the complete streams entering `layer`; returns the index of the self.pre buffer that holds
        the collapse weights they go with."""
        lw = self.w.layers[layer]
        pre_idx = self._cur
        if self._sp_active is not None:
            lo, Rl, R = self._sp_active
            ctx = self._sp_gather_ctx(Rl)
            self._sp_hc(lo, Rl, self._sp_pending, lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, lw.attn_norm,
                        ctx["views"][ctx["parity"]][lo:])
            self._sp_pending = None
            if lw.ratio and sources:
                self._sp_qkv(layer, lw, R, Rl, self._inv(layer), True, ctx)
            return pre_idx
        self._hc(rows, getattr(self, "_pending", None), lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, lw.attn_norm)
        self._pending = None
        if lw.ratio and sources:
            self._qkv(layer, lw, rows, self._inv(layer), True)
        return pre_idx

    def prefill_ced(self, slot: int, tokens: List[int], start: int = 0, chunk: Optional[int] = None) -> int:
        """Prompt pass with the decoder layers replayed for the tail only: layers below cfg.ced_boundary run over every
        chunk and the boundary layer produces its compressed source for every token; the layers from the boundary
        upwards then run over the last cfg.ced_replay tokens, whose streams were kept at the boundary.  Falls back to
        prefill() when the model has no usable boundary or when a continuation is shorter than the replay span (its
        decoder windows must then be continued, not rebuilt).  Returns the greedy next token.
        Reference: rust/crates/ds41rt-daemon/src/v41_backbone_cache/ced.rs:3-34,
        rust/crates/ds41rt-daemon/src/v41_native_serve.rs:620-738."""
        cfg = self.cfg
        n = len(tokens)
        if not self.ced_usable(start, n):
            return self.prefill(slot, tokens, start, chunk)
        chunk = chunk or self.max_rows
        end = start + n
        assert self.cache.ensure(slot, end + 1)
        r0 = self.ced_replay_start(start, end)
        for c0 in range(start, end, chunk):
            c1 = min(end, c0 + chunk)
            self.set_rows(tokens[c0 - start:c1 - start], list(range(c0, c1)), [slot] * (c1 - c0))
            self.ced_encoder_slice(c0, c1, r0)
        nxt = -1
        for c0 in range(r0, end, chunk):
            c1 = min(end, c0 + chunk)
            self.set_rows(tokens[c0 - start:c1 - start], list(range(c0, c1)), [slot] * (c1 - c0),
                          row_lo=[r0] * (c1 - c0))
            self.ced_replay_slice(c0, c1, r0, head=c1 >= end)
            if c1 >= end:
                nxt = int(self.chosen[self.last_head_row].item())
        return nxt

    def ced_usable(self, start: int, n_new: int) -> bool:
        """Can a prompt pass of `n_new` tokens from position `start` use the encoder / replay split?  A continuation
        shorter than the replay span must continue the decoder windows instead of rebuilding them."""
        cfg = self.cfg
        return cfg.ced_on and n_new > 0 and (start == 0 or n_new >= cfg.ced_replay) \
            and not any(l >= cfg.ced_boundary for l in self.engram)

    def ced_replay_start(self, start: int, end: int) -> int:
        return max(start, end - self.cfg.ced_replay)

    def ced_encoder_slice(self, c0: int, c1: int, r0: int, sources: bool = True):
        """Rows set by set_rows() are prompt positions [c0, c1): run the layers below the boundary, produce the boundary
        layer's compressed source, and keep the boundary streams of the positions >= r0 for the replay.
        sources=False: the compressed rows of these positions are already in the cache (restored pages)."""
        cfg = self.cfg
        B, m = cfg.ced_boundary, c1 - c0
        if getattr(self, "ced_streams", None) is None:
            self.ced_streams = torch.zeros(cfg.ced_replay, cfg.hc_mult, cfg.hidden, dtype=BF16, device=self.device)
            self.ced_pre = torch.zeros(cfg.ced_replay, cfg.hc_mult, dtype=F32, device=self.device)
        self.forward_rows(self.sp_rows(m), head=False, last_layer=B, sources=sources)
        pre_idx = self.boundary_source(m, B, sources)
        lo = max(c0, r0)
        if self._sp_active is not None:
            # the streams are row-sharded: every rank contributes the kept rows it owns, the sum assembles them
            own0, Rl, _ = self._sp_active
            self._sp_active = None
            if lo < c1:
                ks, kp = self.ced_streams[lo - r0:c1 - r0], self.ced_pre[lo - r0:c1 - r0]
                ks.zero_()
                kp.zero_()
                a, b = max(lo - c0, own0), min(m, own0 + Rl)
                if a < b:
                    ks[a - (lo - c0):b - (lo - c0)].copy_(self.streams[a:b])
                    kp[a - (lo - c0):b - (lo - c0)].copy_(self.pre[pre_idx][a:b])
                if self.world > 1:
                    import torch.distributed as dist
                    dist.all_reduce(ks, group=self.fabric.group)
                    dist.all_reduce(kp, group=self.fabric.group)
        elif lo < c1:
            self.ced_streams[lo - r0:c1 - r0].copy_(self.streams[lo - c0:m])
            self.ced_pre[lo - r0:c1 - r0].copy_(self.pre[pre_idx][lo - c0:m])

    def ced_replay_slice(self, c0: int, c1: int, r0: int, head: bool):
        """Rows set by set_rows() are prompt positions [c0, c1) of the replayed tail: continue them from the kept
        boundary streams through the layers from the boundary upwards (compressed sources stay as they are)."""
        m = c1 - c0
        self._cur, self._ccur, self._pending, self._cand_ratio, self._sp_active = 0, 0, None, None, None
        self.streams[:m].copy_(self.ced_streams[c0 - r0:c1 - r0])
        self.pre[0][:m].copy_(self.ced_pre[c0 - r0:c1 - r0])
        self.forward_rows(m, embed=False, head=head, first_layer=self.cfg.ced_boundary, sources=False)

    def logits_rows(self, rows: int) -> torch.Tensor:
        """Full-vocabulary fp32 logits of the last pass (gathers vocabulary shards over the process group)."""
        local = self.logits[:rows].clone()
        if self.world == 1:
            return local
        import torch.distributed as dist
        parts = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(parts, local, group=self.fabric.group)
        return torch.cat(parts, dim=1)

    def check_status(self, what: str = "engine pass"):
        lib.raise_on_status(self.status, what)
