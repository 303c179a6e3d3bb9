"""CPU fp32 oracle for the DS41 architecture (full-sequence, cache-free).

Every GPU kernel and the incremental engine are checked against this file.  It
restates the model mathematics extracted from the reference's kernels:

* hyper-connections      native/cuda/kernels/v41_hc.cu:6-29,70-120 (mixes, collapse, expand)
* norms / RoPE           native/cuda/kernels/v41_attention_ops.cu:24-68,328-341
* compressor pooling     native/cuda/kernels/v41_compressor.cu:69-108
* lightning indexer      native/cuda/kernels/v41_index_scores.cu:36-103
* sparse attention+sink  native/cuda/kernels/v41_sparse_attention.cu:216,295
* router                 native/cuda/kernels/v41_router.cu:13-112
* clamp-SwiGLU experts   native/cuda/kernels/v41_fp8.cu:14-21, docs/ds41-expert-qualification.md:5-11

The whole prompt is processed at once with explicit causal masks, so a token's
result depends only on earlier tokens exactly as in incremental decoding.
Optional `kv_quant=True` applies the cache formats' quantise/dequantise
round trips (FP8+UE8M0/32 window rows, FP4+E4M3/16 compressed rows, FP4+UE8M0/32
index keys and queries) so cache-format effects can be compared too.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..config import ModelConfig, RopeConfig, rope_inv_freq
from ..ops import quant_ref as Q


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)
    return y * w.float() if w is not None else y


def apply_rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, rope_dim: int,
               inverse: bool = False) -> torch.Tensor:
    """Rotate adjacent pairs of the last `rope_dim` dims of x[..., D] by pos * inv_freq.
    `pos` has x's leading shape minus any head axis (broadcast over heads)."""
    if rope_dim == 0:
        return x
    head = x[..., : x.shape[-1] - rope_dim]
    tail = x[..., x.shape[-1] - rope_dim:]
    ang = pos.to(torch.float32)[..., None] * inv_freq.to(torch.float32)
    while ang.dim() < tail.dim():
        ang = ang.unsqueeze(-2)
    c, s = torch.cos(ang), torch.sin(ang)
    if inverse:
        s = -s
    a, b = tail[..., 0::2], tail[..., 1::2]
    ra = a * c - b * s
    rb = b * c + a * s
    return torch.cat([head, torch.stack([ra, rb], -1).flatten(-2)], -1)


def hc_mixes(streams: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor,
             mult: int, iters: int, hc_eps: float, norm_eps: float):
    """streams [T, mult, H] -> (pre [T,mult], post [T,mult], comb [T,mult,mult] indexed [s,d])."""
    T = streams.shape[0]
    flat = streams.reshape(T, -1).float()
    inv = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + norm_eps)
    proj = (flat @ fn.float().t()) * inv                                     # [T, 2m+m^2]
    pre = torch.sigmoid(proj[:, :mult] * scale[0] + base[:mult]) + hc_eps
    post = 2.0 * torch.sigmoid(proj[:, mult:2 * mult] * scale[1] + base[mult:2 * mult])
    c = (proj[:, 2 * mult:] * scale[2] + base[2 * mult:]).view(T, mult, mult)  # [s, d]
    c = torch.softmax(c, dim=2) + hc_eps                                      # rows (over d)
    c = c / (c.sum(dim=1, keepdim=True) + hc_eps)                             # columns (over s)
    for _ in range(iters - 1):
        c = c / (c.sum(dim=2, keepdim=True) + hc_eps)
        c = c / (c.sum(dim=1, keepdim=True) + hc_eps)
    return pre, post, c


def hc_collapse(streams: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    return torch.einsum("ts,tsh->th", pre, streams.float())


def hc_expand(streams: torch.Tensor, sub: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    return post[:, :, None] * sub[:, None, :].float() + torch.einsum("tsd,tsh->tdh", comb, streams.float())


def router(x: torch.Tensor, gate_w: torch.Tensor, bias: torch.Tensor, topk: int, route_scale: float):
    """Returns (expert ids [T,k] ordered by descending biased score, weights [T,k])."""
    logits = x.float() @ gate_w.float().t()
    score = torch.sqrt(F.softplus(logits))
    biased = score + bias.float()
    order = torch.sort(biased, dim=-1, descending=True, stable=True).indices[:, :topk]
    sel = torch.gather(score, 1, order)
    w = sel / (sel.sum(-1, keepdim=True) + 1e-20) * route_scale
    return order, w


def swiglu_clamped(gate: torch.Tensor, up: torch.Tensor, limit: float) -> torch.Tensor:
    gate = gate.clamp(max=limit)
    up = up.clamp(min=-limit, max=limit)
    return F.silu(gate) * up


def expert_ffn(x, w1, w3, w2, limit, route_w=None, act_qdq=None):
    """act_qdq = (f_in, f_mid): optional quantise-dequantise of the FC1 and FC2 inputs (W4A4 / W8A8 expert variants)."""
    if act_qdq is not None:
        x = act_qdq[0](x)
    act = swiglu_clamped(x @ w1.float().t(), x @ w3.float().t(), limit)
    if route_w is not None:
        act = act * route_w[:, None]          # route weight is applied before FC2
    if act_qdq is not None:
        act = act_qdq[1](act.bfloat16().float())
    return act @ w2.float().t()


@dataclass
class LayerTrace:
    """Intermediate values kept for kernel-level tests."""
    x_attn_norm: torch.Tensor = None
    q: torch.Tensor = None
    kv: torch.Tensor = None
    comp: Optional[torch.Tensor] = None
    index_keys: Optional[torch.Tensor] = None
    select: Optional[torch.Tensor] = None
    attn_out: torch.Tensor = None
    experts: torch.Tensor = None
    route_w: torch.Tensor = None
    streams_out: torch.Tensor = None
    x_ffn_norm: torch.Tensor = None
    moe_out: torch.Tensor = None
    route_logits: torch.Tensor = None


class ReferenceModel:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], kv_quant: bool = False):
        self.cfg = cfg
        self.w = weights
        self.kv_quant = kv_quant
        self._inv = {}

    # ------------------------------------------------------------------ helpers
    engram_hook = None   # optional callable (layer, streams [T, m, H]) -> streams, applied on entry to each layer

    def inv_freq(self, rope: RopeConfig, dim: int) -> torch.Tensor:
        key = (rope.theta, rope.factor, dim)
        if key not in self._inv:
            self._inv[key] = torch.tensor(rope_inv_freq(rope, dim), dtype=torch.float32)
        return self._inv[key]

    def _g(self, name: str) -> torch.Tensor:
        return self.w[name].float()

    # ------------------------------------------------------------------ pieces
    def compress_source(self, p: str, layer: int, xn: torch.Tensor, positions: torch.Tensor):
        """Compressed latents + index keys produced by source layer `layer` from the
        attn-normalised hidden of all T tokens.  Returns (comp [Tc,D] roped, index_keys
        [Tc,ID] roped, first_pos [Tc])."""
        cfg = self.cfg
        ratio = cfg.source_layers[layer]
        rope = cfg.rope_for(layer)
        kv = xn @ self._g(f"{p}.attn.compressor.wkv.weight").t()
        T = xn.shape[0]
        if ratio == 2:
            gate = xn @ self._g(f"{p}.attn.compressor.wgate.weight").t()
            Tc = T // 2
            kv2 = kv[: Tc * 2].view(Tc, 2, -1)
            g2 = gate[: Tc * 2].view(Tc, 2, -1)
            wgt = torch.softmax(g2, dim=1)
            pooled = (wgt * kv2).sum(1)
            first = positions[: Tc * 2: 2]
        else:
            Tc = T
            pooled = kv
            first = positions
        latent = rmsnorm(pooled, self._g(f"{p}.attn.compressor.norm.weight"), cfg.norm_eps)
        ik = latent @ self._g(f"{p}.attn.indexer.wk.weight").t()
        ik = rmsnorm(ik, self._g(f"{p}.attn.indexer.k_norm.weight"), cfg.norm_eps)
        ik = apply_rope(ik, first, self.inv_freq(rope, cfg.index_dim // 2), cfg.index_dim // 2)
        comp = apply_rope(latent, first, self.inv_freq(rope, cfg.rope_dim), cfg.rope_dim)
        if self.kv_quant:
            ik = Q.qdq_mxfp4(ik, 32) if cfg.index_dim % 32 == 0 else ik
            p4, bs = Q.quant_kv_fp4_e4m3_16(comp)
            comp = Q.dequant_kv_fp4_e4m3_16(p4, bs)
        return comp, ik, first

    def index_scores(self, p: str, layer: int, q_lat: torch.Tensor, xn: torch.Tensor,
                     positions: torch.Tensor, index_keys: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        rope = cfg.rope_for(layer)
        T = q_lat.shape[0]
        iq = (q_lat @ self._g(f"{p}.attn.indexer.wq_b.weight").t()).view(T, cfg.index_heads, cfg.index_dim)
        iq = apply_rope(iq, positions, self.inv_freq(rope, cfg.index_dim // 2), cfg.index_dim // 2)
        if self.kv_quant and cfg.index_dim % 32 == 0:
            iq = Q.qdq_mxfp4(iq, 32)
        wts = (xn @ self._g(f"{p}.attn.indexer.weights_proj.weight").t()) * cfg.index_weight_scale
        dots = torch.relu(torch.einsum("thd,cd->thc", iq, index_keys))
        return torch.einsum("th,thc->tc", wts, dots)

    def select_topk(self, scores: torch.Tensor, visible: torch.Tensor, k: int) -> torch.Tensor:
        """scores [T,Tc], visible bool [T,Tc] -> bool mask of the top-k visible rows
        (all visible rows when there are at most k); ties favour the lower row."""
        masked = scores.masked_fill(~visible, float("-inf"))
        order = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :k]
        sel = torch.zeros_like(visible)
        sel.scatter_(1, order, True)
        return sel & visible

    def attention(self, p: str, layer: int, xn: torch.Tensor, positions: torch.Tensor,
                  source, select: Optional[torch.Tensor], trace: Optional[LayerTrace] = None,
                  attend_all_draft: int = 0, kv_prefix: Optional[torch.Tensor] = None,
                  prefix_pos: Optional[torch.Tensor] = None):
        """Sparse latent attention for all T query rows.  `source` = (comp, first_pos, ratio) or None."""
        cfg = self.cfg
        T = xn.shape[0]
        rope = cfg.rope_for(layer) if p.startswith("layers") else cfg.rope_plain
        inv = self.inv_freq(rope, cfg.rope_dim)
        q_lat = rmsnorm(xn @ self._g(f"{p}.attn.wq_a.weight").t(), self._g(f"{p}.attn.q_norm.weight"), cfg.norm_eps)
        q = (q_lat @ self._g(f"{p}.attn.wq_b.weight").t()).view(T, cfg.n_heads, cfg.head_dim)
        q = apply_rope(q, positions, inv, cfg.rope_dim)
        kv = rmsnorm(xn @ self._g(f"{p}.attn.wkv.weight").t(), self._g(f"{p}.attn.kv_norm.weight"), cfg.norm_eps)
        kv = apply_rope(kv, positions, inv, cfg.rope_dim)
        if self.kv_quant:
            kv = Q.qdq_mxfp8(kv, 32)
        if trace is not None:
            trace.q, trace.kv = q, kv
        # window keys (optionally preceded by externally produced rows, e.g. the drafter's committed ring)
        key_pos = positions
        if kv_prefix is not None:
            kv = torch.cat([kv_prefix.float(), kv], 0)
            key_pos = torch.cat([prefix_pos, positions])
        pj = key_pos[None, :]
        pt = positions[:, None]
        hi = pt.clone()
        if attend_all_draft:
            # drafter rows: the last `attend_all_draft` rows see each other non-causally
            hi[-attend_all_draft:] = positions[-1]
        wmask = (pj <= hi) & (pj > pt - cfg.window)
        logits = torch.einsum("thd,jd->thj", q, kv) * cfg.softmax_scale
        logits = logits.masked_fill(~wmask[:, None, :], float("-inf"))
        values = kv
        if source is not None and select is not None:
            comp = source[0]
            lc = torch.einsum("thd,cd->thc", q, comp) * cfg.softmax_scale
            lc = lc.masked_fill(~select[:, None, :], float("-inf"))
            logits = torch.cat([logits, lc], -1)
            values = torch.cat([kv, comp], 0)
        sink = self._g(f"{p}.attn.attn_sink")[None, :, None]
        m = torch.maximum(logits.amax(-1, keepdim=True), sink)
        e = torch.exp(logits - m)
        denom = e.sum(-1, keepdim=True) + torch.exp(sink - m)
        out = torch.einsum("thj,jd->thd", e / denom, values)
        out = apply_rope(out, positions, inv, cfg.rope_dim, inverse=True)
        # grouped output projection
        G, hpg = cfg.o_groups, cfg.heads_per_group
        wo_a = self._g(f"{p}.attn.wo_a.weight").view(G, cfg.o_lora, hpg * cfg.head_dim)
        og = torch.einsum("tgk,gok->tgo", out.reshape(T, G, hpg * cfg.head_dim), wo_a).reshape(T, G * cfg.o_lora)
        res = og @ self._g(f"{p}.attn.wo_b.weight").t()
        if trace is not None:
            trace.attn_out = res
        return res, q_lat

    def moe(self, p: str, xn: torch.Tensor, n_experts: int, topk: int, trace: Optional[LayerTrace] = None):
        cfg = self.cfg
        ids, wts = router(xn, self._g(f"{p}.ffn.gate.weight"), self._g(f"{p}.ffn.gate.bias"), topk, cfg.route_scale)
        out = torch.zeros(xn.shape[0], cfg.hidden)
        for e in range(n_experts):
            hit = (ids == e)
            rows = hit.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            rw = (wts * hit)[rows].sum(-1)
            out[rows] += expert_ffn(xn[rows], self._g(f"{p}.ffn.experts.{e}.w1.weight"),
                                    self._g(f"{p}.ffn.experts.{e}.w3.weight"),
                                    self._g(f"{p}.ffn.experts.{e}.w2.weight"), cfg.swiglu_limit, rw,
                                    getattr(self, "expert_act_qdq", None))
        out = out + expert_ffn(xn, self._g(f"{p}.ffn.shared_experts.w1.weight"),
                               self._g(f"{p}.ffn.shared_experts.w3.weight"),
                               self._g(f"{p}.ffn.shared_experts.w2.weight"), cfg.swiglu_limit)
        if trace is not None:
            trace.experts, trace.route_w = ids, wts
        return out

    def block(self, p: str, layer: int, streams, pre, positions, source, select, n_experts, topk,
              trace=None, attend_all_draft: int = 0, produce=None, kv_prefix=None, prefix_pos=None):
        """One decoder block on streams [T,m,H] with incoming pre [T,m].
        `produce(xn, q_lat)` lets the caller build sources/selections from this layer's
        normalised input before attention runs; it returns (source, select)."""
        cfg = self.cfg
        mix = lambda s, kind: hc_mixes(s, self._g(f"{p}.hc_{kind}_fn"), self._g(f"{p}.hc_{kind}_scale"),
                                       self._g(f"{p}.hc_{kind}_base"), cfg.hc_mult, cfg.hc_sinkhorn_iters,
                                       cfg.hc_eps, cfg.norm_eps)
        next_pre, post, comb = mix(streams, "attn")
        xn = rmsnorm(hc_collapse(streams, pre), self._g(f"{p}.attn_norm.weight"), cfg.norm_eps)
        if trace is not None:
            trace.x_attn_norm = xn
        if produce is not None:
            source, select = produce(xn)
        a, _ = self.attention(p, layer, xn, positions, source, select, trace, attend_all_draft, kv_prefix,
                              prefix_pos)
        streams = hc_expand(streams, a, post, comb)
        pre = next_pre
        next_pre, post, comb = mix(streams, "ffn")
        xn = rmsnorm(hc_collapse(streams, pre), self._g(f"{p}.ffn_norm.weight"), cfg.norm_eps)
        f = self.moe(p, xn, n_experts, topk, trace)
        streams = hc_expand(streams, f, post, comb)
        if trace is not None:
            trace.streams_out = streams
            trace.x_ffn_norm, trace.moe_out = xn, f
            trace.route_logits = xn @ self._g(f"{p}.ffn.gate.weight").t()
        return streams, next_pre

    # ------------------------------------------------------------------ full forward
    def forward(self, tokens: torch.Tensor, return_trace: bool = False, return_taps: bool = False):
        """tokens [T] -> logits [T, vocab] (fp32)."""
        cfg = self.cfg
        T = tokens.shape[0]
        positions = torch.arange(T)
        h = self._g("embed.weight")[tokens]
        streams = h[:, None, :].repeat(1, cfg.hc_mult, 1)
        pre = torch.zeros(T, cfg.hc_mult)
        pre[:, 0] = 1.0
        sources: Dict[int, tuple] = {}
        selections: Dict[int, torch.Tensor] = {}
        candidates: Optional[torch.Tensor] = None
        traces: List[LayerTrace] = []
        taps = []
        for l in range(cfg.n_layers):
            p = f"layers.{l}"
            tr = LayerTrace() if return_trace else None
            if self.engram_hook is not None:
                # Engram memory: layers that have one update the streams they receive (bf16 rounding as the kernel)
                streams = self.engram_hook(l, streams)
            if cfg.dspark is not None and l in cfg.dspark.tap_layers:
                taps.append(streams.mean(1))
            src_layer = cfg.source_of(l)

            def produce(xn, l=l, p=p, src_layer=src_layer, tr=tr):
                nonlocal candidates
                if src_layer is None:
                    return None, None
                if l in cfg.source_layers:
                    comp, ik, first = self.compress_source(p, l, xn, positions)
                    sources[l] = (comp, first, cfg.source_layers[l], ik)
                comp, first, ratio, ik = sources[src_layer]
                Tc = comp.shape[0]
                n_vis = (positions + 1) // ratio
                visible = torch.arange(Tc)[None, :] < n_vis[:, None]
                if l in cfg.index_layers:
                    q_lat = rmsnorm(xn @ self._g(f"{p}.attn.wq_a.weight").t(),
                                    self._g(f"{p}.attn.q_norm.weight"), cfg.norm_eps)
                    sc = self.index_scores(p, l, q_lat, xn, positions, ik)
                    vis = visible
                    if cfg.candidate_layer >= 0 and cfg.candidate_topk_blocks > 0:
                        if l == cfg.candidate_layer:
                            candidates = self._candidate_blocks(sc, visible)
                        elif l > cfg.candidate_layer and candidates is not None:
                            vis = visible & candidates
                    selections[l] = self.select_topk(sc, vis, cfg.index_topk)
                sel = selections[cfg.index_producer_of(l)]
                if tr is not None:
                    tr.comp, tr.index_keys, tr.select = comp, ik, sel
                return (comp, first, ratio), sel

            streams, pre = self.block(p, l, streams, pre, positions, None, None, cfg.n_experts, cfg.topk,
                                      tr, produce=produce)
            if return_trace:
                traces.append(tr)
        x = rmsnorm(hc_collapse(streams, pre), self._g("norm.weight"), cfg.norm_eps)
        logits = x @ self._g("head.weight").t()
        out = [logits]
        if return_trace:
            out.append(traces)
        if return_taps:
            out.append(taps)
        return out[0] if len(out) == 1 else tuple(out)

    def forward_ced(self, tokens: torch.Tensor, boundary: int, replay: int = 128) -> torch.Tensor:
        """Prefill with the decoder layers replayed only for the prompt's tail (reference:
        rust/crates/ds41rt-daemon/src/v41_backbone_cache/ced.rs:3-34, docs/ds41-ced-cache-transactions.md:8-20).
        Layers [0, boundary) run over all tokens and layer `boundary` produces its compressed source from all of them;
        layers [boundary, n_layers) then run only over the last `replay` tokens: their windows hold those tokens only,
        the compressed sources are complete.  Returns the logits of the replayed rows [min(replay, T), vocab]."""
        cfg = self.cfg
        T = tokens.shape[0]
        assert 0 < boundary < cfg.n_layers and all(s <= boundary for s in cfg.source_layers if s < cfg.n_layers)
        positions = torch.arange(T)
        streams = self._g("embed.weight")[tokens][:, None, :].repeat(1, cfg.hc_mult, 1)
        pre = torch.zeros(T, cfg.hc_mult)
        pre[:, 0] = 1.0
        sources: Dict[int, tuple] = {}
        selections: Dict[int, torch.Tensor] = {}
        candidates: Optional[torch.Tensor] = None

        def make_produce(l, pos, recompute):
            p = f"layers.{l}"
            src_layer = cfg.source_of(l)

            def produce(xn):
                nonlocal candidates
                if src_layer is None:
                    return None, None
                if l in cfg.source_layers and recompute:
                    comp, ik, first = self.compress_source(p, l, xn, pos)
                    sources[l] = (comp, first, cfg.source_layers[l], ik)
                comp, first, ratio, ik = sources[src_layer]
                visible = torch.arange(comp.shape[0])[None, :] < ((pos + 1) // ratio)[:, None]
                if l in cfg.index_layers:
                    q_lat = rmsnorm(xn @ self._g(f"{p}.attn.wq_a.weight").t(), self._g(f"{p}.attn.q_norm.weight"),
                                    cfg.norm_eps)
                    sc = self.index_scores(p, l, q_lat, xn, pos, ik)
                    vis = visible
                    if cfg.candidate_layer >= 0 and cfg.candidate_topk_blocks > 0:
                        if l == cfg.candidate_layer:
                            candidates = self._candidate_blocks(sc, visible)
                        elif l > cfg.candidate_layer and candidates is not None:
                            vis = visible & candidates
                    selections[l] = self.select_topk(sc, vis, cfg.index_topk)
                return (comp, first, ratio), selections[cfg.index_producer_of(l)]
            return produce

        for l in range(boundary):
            if self.engram_hook is not None:
                streams = self.engram_hook(l, streams)
            streams, pre = self.block(f"layers.{l}", l, streams, pre, positions, None, None, cfg.n_experts, cfg.topk,
                                      None, produce=make_produce(l, positions, True))
        pb = f"layers.{boundary}"
        if boundary in cfg.source_layers:
            xn = rmsnorm(hc_collapse(streams, pre), self._g(f"{pb}.attn_norm.weight"), cfg.norm_eps)
            comp, ik, first = self.compress_source(pb, boundary, xn, positions)
            sources[boundary] = (comp, first, cfg.source_layers[boundary], ik)
        s0 = max(0, T - replay)
        streams, pre, pos = streams[s0:], pre[s0:], positions[s0:]
        candidates = None
        for l in range(boundary, cfg.n_layers):
            streams, pre = self.block(f"layers.{l}", l, streams, pre, pos, None, None, cfg.n_experts, cfg.topk,
                                      None, produce=make_produce(l, pos, False))
        x = rmsnorm(hc_collapse(streams, pre), self._g("norm.weight"), cfg.norm_eps)
        return x @ self._g("head.weight").t()

    def _candidate_blocks(self, scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
        """Top candidate blocks of `candidate_block` rows by block-max score; the newest
        visible block is always kept (native/cuda/kernels/v41_candidate_blocks.cu:18-44)."""
        cfg = self.cfg
        T, Tc = scores.shape
        B = cfg.candidate_block
        nb = (Tc + B - 1) // B
        s = scores.masked_fill(~visible, float("-inf"))
        s = F.pad(s, (0, nb * B - Tc), value=float("-inf")).view(T, nb, B).amax(-1)
        n_vis = visible.sum(-1)
        newest = ((n_vis - 1).clamp(min=0) // B)
        s.scatter_(1, newest[:, None], float("inf"))
        order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, : cfg.candidate_topk_blocks]
        keep = torch.zeros(T, nb, dtype=torch.bool)
        keep.scatter_(1, order, True)
        return keep.repeat_interleave(B, 1)[:, :Tc]

    # ------------------------------------------------------------------ dSpark drafter
    def dspark_main(self, taps: List[torch.Tensor]) -> torch.Tensor:
        """Tap means [T,H] of the tap layers -> normalised conditioning rows [T,H]."""
        x = torch.cat([t.float() for t in taps], -1) @ self._g("mtp.0.main_proj.weight").t()
        return rmsnorm(x, self._g("mtp.0.main_norm.weight"), self.cfg.norm_eps)

    @torch.no_grad()
    def dspark_draft(self, main: torch.Tensor, anchor: int, width: int):
        """Draft `width` tokens following `anchor` given conditioning rows for positions 0..T-1.
        Returns (draft tokens [width], base logits [width, vocab])."""
        cfg, d = self.cfg, self.cfg.dspark
        T = main.shape[0]
        toks = torch.tensor([anchor] + [d.noise_token_id] * (width - 1))
        positions = torch.arange(T, T + width)
        prefix_pos = torch.arange(T)
        inv = self.inv_freq(cfg.rope_plain, cfg.rope_dim)
        streams = self._g("embed.weight")[toks][:, None, :].repeat(1, cfg.hc_mult, 1)
        pre = torch.zeros(width, cfg.hc_mult)
        pre[:, 0] = 1.0
        saved_window = cfg.window
        cfg.window = d.ring_rows
        try:
            for s in range(d.stages):
                p = f"mtp.{s}"
                kvp = rmsnorm(main @ self._g(f"{p}.attn.wkv.weight").t(), self._g(f"{p}.attn.kv_norm.weight"),
                              cfg.norm_eps)
                kvp = apply_rope(kvp, prefix_pos, inv, cfg.rope_dim)
                streams, pre = self.block(p, -1, streams, pre, positions, None, None, d.n_experts, d.topk,
                                          attend_all_draft=width, kv_prefix=kvp, prefix_pos=prefix_pos)
        finally:
            cfg.window = saved_window
        last = d.stages - 1
        x = rmsnorm(hc_collapse(streams, pre), self._g(f"mtp.{last}.norm.weight"), cfg.norm_eps)
        logits = x @ self._g("head.weight").t()
        me, mh = self._g(f"mtp.{last}.markov_head.embed.weight"), self._g(f"mtp.{last}.markov_head.head.weight")
        drafts, prev = [], anchor
        for j in range(width):
            lj = logits[j] + mh @ me[prev]
            prev = int(torch.argmax(lj))
            drafts.append(prev)
        return torch.tensor(drafts), logits

    @torch.no_grad()
    def generate_greedy(self, prompt: torch.Tensor, n_new: int):
        """Greedy decode by re-running the full forward (oracle simplicity over speed).
        Returns (tokens [n_new], logits [n_new, vocab])."""
        toks = prompt.clone()
        outs, logs = [], []
        for _ in range(n_new):
            logits = self.forward(toks)[-1]
            nxt = int(torch.argmax(logits))
            outs.append(nxt)
            logs.append(logits)
            toks = torch.cat([toks, torch.tensor([nxt])])
        return torch.tensor(outs), torch.stack(logs)
