"""Vision tower (ViT) and aligner on the GPU kernels: image patches -> rows for the language model's embedding stream.

Structure (tensor names as in the checkpoint catalog, `loader/catalog.py`): patch projection (+bias) -> `layers` blocks of
[RMSNorm -> qkv (+bias) -> 2-D RoPE -> bidirectional attention -> wo (+bias) -> residual; RMSNorm -> SwiGLU MLP ->
residual] -> RMSNorm -> 3x3 merge -> aligner (linear + GELU + linear).  Every projection and both attention products
run on the tcgen05 GEMM (`ops/gemm.py`); the kernels between them are in csrc/kernels/vision.cu.  Attention is done per
query tile: S = Q K^T for all heads in one batched launch, a row softmax, then P V against V^T (which the value
projection produces directly by computing W_v x^T); the value bias is added after attention (softmax rows sum to one).

`vision_reference` is the plain PyTorch fp32 statement of the same network for tests.
Reference: 32-layer ViT, 1024 wide, 16 heads, patch 14, 2-D RoPE, 3x3 merge, GELU aligner to 5120
(rust/crates/ds41rt-loader/src/v41_config.rs:157-169, native/include/ds41rt_v41_vision.h:7-45, native/cuda/kernels/v41_vision.cu).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Tuple

import torch

from ..config import VisionConfig
from ..ops import gemm as G
from ..ops import lib

BF16 = torch.bfloat16


def init_vision_weights(v: VisionConfig, hidden: int, layers: int, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = v.hidden
    r = lambda *s: torch.randn(*s, generator=g) * std
    w = {"vision.patch_embed.proj.weight": r(W, 3 * v.patch * v.patch), "vision.patch_embed.proj.bias": r(W),
         "vision.norm.weight": torch.ones(W) + r(W), "aligner.w1.weight": r(hidden, W * v.downsample ** 2),
         "aligner.w1.bias": r(hidden), "aligner.w2.weight": r(hidden, hidden), "aligner.w2.bias": r(hidden)}
    for b in range(layers):
        p = f"vision.blocks.{b}"
        w.update({f"{p}.attn.wqkv.weight": r(3 * W, W), f"{p}.attn.wqkv.bias": r(3 * W), f"{p}.attn.wo.weight": r(W, W),
                  f"{p}.attn.wo.bias": r(W), f"{p}.mlp.w1.weight": r(2 * v.intermediate, W),
                  f"{p}.mlp.w2.weight": r(W, v.intermediate), f"{p}.norm1.weight": torch.ones(W) + r(W),
                  f"{p}.norm2.weight": torch.ones(W) + r(W)})
    return w


def _rope2d_ref(t: torch.Tensor, pos_hw: torch.Tensor, heads: int, theta: float) -> torch.Tensor:
    n, W = t.shape
    d = W // heads
    half = d // 2
    x = t.view(n, heads, d).clone()
    i = torch.arange(half // 2, dtype=torch.float32)
    freq = theta ** (-2.0 * i / half)
    for axis in range(2):
        ang = pos_hw[:, axis:axis + 1].float() * freq[None]            # [n, half/2]
        cs, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        seg = x[:, :, axis * half:(axis + 1) * half]
        a, b = seg[..., 0::2].clone(), seg[..., 1::2].clone()
        seg[..., 0::2] = a * cs - b * sn
        seg[..., 1::2] = b * cs + a * sn
    return x.view(n, W)


def vision_reference(v: VisionConfig, w: Dict[str, torch.Tensor], patches: torch.Tensor, grid: Tuple[int, int],
                     layers: int, eps: float = 1e-6) -> torch.Tensor:
    """patches [gh*gw, 3*patch*patch] fp32 -> [gh*gw / downsample^2, hidden] fp32."""
    gh, gw = grid
    n, W, heads = gh * gw, v.hidden, v.heads
    pos = torch.stack(torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij"), -1).view(n, 2)
    rms = lambda t, g: t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * g
    x = patches @ w["vision.patch_embed.proj.weight"].t() + w["vision.patch_embed.proj.bias"]
    for b in range(layers):
        p = f"vision.blocks.{b}"
        qkv = rms(x, w[f"{p}.norm1.weight"]) @ w[f"{p}.attn.wqkv.weight"].t() + w[f"{p}.attn.wqkv.bias"]
        q = _rope2d_ref(qkv[:, :W], pos, heads, v.rope_theta).view(n, heads, -1).transpose(0, 1)
        k = _rope2d_ref(qkv[:, W:2 * W], pos, heads, v.rope_theta).view(n, heads, -1).transpose(0, 1)
        val = qkv[:, 2 * W:].view(n, heads, -1).transpose(0, 1)
        att = torch.softmax(q @ k.transpose(1, 2) / math.sqrt(W // heads), -1) @ val
        x = x + att.transpose(0, 1).reshape(n, W) @ w[f"{p}.attn.wo.weight"].t() + w[f"{p}.attn.wo.bias"]
        gu = rms(x, w[f"{p}.norm2.weight"]) @ w[f"{p}.mlp.w1.weight"].t()
        I = v.intermediate
        x = x + (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]) @ w[f"{p}.mlp.w2.weight"].t()
    x = rms(x, w["vision.norm.weight"])
    m = v.downsample
    x = x.view(gh // m, m, gw // m, m, W).permute(0, 2, 1, 3, 4).reshape((gh // m) * (gw // m), m * m * W)
    h = torch.nn.functional.gelu(x @ w["aligner.w1.weight"].t() + w["aligner.w1.bias"])
    return h @ w["aligner.w2.weight"].t() + w["aligner.w2.bias"]


class VisionTower:
    def __init__(self, v: VisionConfig, weights: Dict[str, torch.Tensor], hidden: int, layers: int, device,
                 max_patches: int = 9216, query_tile: int = 1024, eps: float = 1e-6):
        self.v, self.H, self.layers, self.dev, self.eps = v, hidden, layers, device, eps
        self.W, self.heads, self.I = v.hidden, v.heads, v.intermediate
        self.kp = (3 * v.patch * v.patch + 7) // 8 * 8                 # patch vector padded to a 16-byte multiple
        d = lambda t: t.to(device=device, dtype=BF16).contiguous()
        pw = torch.zeros(self.W, self.kp)
        pw[:, :3 * v.patch * v.patch] = weights["vision.patch_embed.proj.weight"]
        self.w = {k: d(t) for k, t in weights.items()}
        self.w["vision.patch_embed.proj.weight"] = d(pw)
        self.max_patches, self.tq = max_patches, query_tile
        n, W = max_patches, self.W
        z = lambda *s, dt=BF16: torch.zeros(*s, dtype=dt, device=device)
        self.n_pad_max = (n + 63) // 64 * 64
        self.x, self.xn, self.qkv, self.att = z(n, W), z(n, W), z(n, 3 * W), z(n, W)
        self.vt = z(W, self.n_pad_max)
        self.scores = z(self.heads, min(self.tq, n), self.n_pad_max, dt=torch.float32)
        self.probs = z(self.heads, min(self.tq, n), self.n_pad_max)
        self.gu, self.act = z(n, 2 * self.I), z(n, self.I)
        m2 = v.downsample ** 2
        self.merged, self.h1, self.out = z(n // m2 + 1, m2 * W), z(n // m2 + 1, hidden), z(n // m2 + 1, hidden)
        self.patches = z(n, self.kp)
        self.pos = torch.zeros(n, 2, dtype=torch.int32, device=device)
        self.status = lib.new_status(device)

    def _lin(self, x, w, out):
        G.matmul_nt(x, w, out, status=self.status)

    def encode(self, patches: torch.Tensor, grid: Tuple[int, int]) -> torch.Tensor:
        """patches [gh*gw, 3*patch*patch] (any float dtype, on any device) -> image rows [gh*gw/9, hidden] bf16."""
        gh, gw = grid
        n, W, heads, k, st = gh * gw, self.W, self.heads, lib.kernels(), lib.stream
        assert patches.shape[0] == n and n <= self.max_patches and gh % self.v.downsample == 0 == gw % self.v.downsample
        d = W // heads
        n_pad = (n + 63) // 64 * 64
        self.patches[:n].zero_()
        self.patches[:n, :patches.shape[1]].copy_(patches.to(self.dev, BF16))
        pos = torch.stack(torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij"), -1).view(n, 2).int()
        self.pos[:n].copy_(pos)
        x, xn, qkv, att = self.x[:n], self.xn[:n], self.qkv[:n], self.att[:n]
        w = self.w
        ck = lambda e, what: lib.check(e, what)
        self._lin(self.patches[:n], w["vision.patch_embed.proj.weight"], x)
        ck(k.ds41_vis_bias_act(lib.ptr(x), lib.ptr(w["vision.patch_embed.proj.bias"]), None, lib.ptr(x),
                               C.c_longlong(n), W, 0, st()), "bias")
        vt = self.vt[:, :n_pad]
        if n_pad > n:
            self.vt.zero_()
        for b in range(self.layers):
            p = f"vision.blocks.{b}"
            ck(k.ds41_vis_rmsnorm(lib.ptr(x), lib.ptr(w[f"{p}.norm1.weight"]), lib.ptr(xn), n, W, C.c_float(self.eps),
                                  st()), "norm1")
            wqkv, bqkv = w[f"{p}.attn.wqkv.weight"], w[f"{p}.attn.wqkv.bias"]
            self._lin(xn, wqkv, qkv)
            ck(k.ds41_vis_bias_act(lib.ptr(qkv), lib.ptr(bqkv), None, lib.ptr(qkv), C.c_longlong(n), 3 * W, 0, st()), "bias")
            ck(k.ds41_vis_rope2d(lib.ptr(qkv), lib.ptr(self.pos), n, W, heads, C.c_float(self.v.rope_theta), st()), "rope")
            # V^T [W, n] = W_v x^T (value bias deferred to after the attention product)
            G.gemm_raw(wqkv[2 * W:], xn, self.vt, W, n, W, lda=W, ldb=W, ldo=self.n_pad_max, out_mode=0,
                       bn=256 if n >= 256 else 64, status=self.status)
            for q0 in range(0, n, self.tq):
                tq = min(self.tq, n - q0)
                qp = qkv[q0:q0 + tq]
                G.gemm_raw(qp, qkv[:, W:], self.scores, tq, n, d, lda=3 * W, ldb=3 * W, ldo=self.n_pad_max, out_mode=1,
                           bn=256 if n >= 256 else 64, batch=heads, a_batch_stride=d, b_batch_stride=d,
                           out_batch_stride=self.scores.stride(0), status=self.status)
                ck(k.ds41_vis_softmax(lib.ptr(self.scores), C.c_longlong(self.n_pad_max),
                                      C.c_longlong(heads * self.scores.shape[1]), n, C.c_float(1.0 / math.sqrt(d)),
                                      lib.ptr(self.probs), C.c_longlong(self.n_pad_max), n_pad, st()), "softmax")
                G.gemm_raw(self.probs, self.vt, att[q0:q0 + tq], tq, d, n_pad, lda=self.n_pad_max, ldb=self.n_pad_max,
                           ldo=W, out_mode=0, bn=64, batch=heads, a_batch_stride=self.probs.stride(0),
                           b_batch_stride=d * self.n_pad_max, out_batch_stride=d, status=self.status)
            ck(k.ds41_vis_bias_act(lib.ptr(att), lib.ptr(bqkv[2 * W:]), None, lib.ptr(att), C.c_longlong(n), W, 0, st()),
               "v bias")
            self._lin(att, w[f"{p}.attn.wo.weight"], xn)
            ck(k.ds41_vis_bias_act(lib.ptr(xn), lib.ptr(w[f"{p}.attn.wo.bias"]), lib.ptr(x), lib.ptr(x), C.c_longlong(n),
                                   W, 0, st()), "wo bias + residual")
            ck(k.ds41_vis_rmsnorm(lib.ptr(x), lib.ptr(w[f"{p}.norm2.weight"]), lib.ptr(xn), n, W, C.c_float(self.eps),
                                  st()), "norm2")
            self._lin(xn, w[f"{p}.mlp.w1.weight"], self.gu[:n])
            ck(k.ds41_vis_silu_mul(lib.ptr(self.gu), lib.ptr(self.act), n, self.I, st()), "silu")
            self._lin(self.act[:n], w[f"{p}.mlp.w2.weight"], xn)
            ck(k.ds41_vis_bias_act(lib.ptr(xn), None, lib.ptr(x), lib.ptr(x), C.c_longlong(n), W, 0, st()), "residual")
        ck(k.ds41_vis_rmsnorm(lib.ptr(x), lib.ptr(w["vision.norm.weight"]), lib.ptr(xn), n, W, C.c_float(self.eps), st()),
           "final norm")
        m = self.v.downsample
        nm = n // (m * m)
        ck(k.ds41_vis_merge(lib.ptr(xn), lib.ptr(self.merged), gh, gw, m, W, st()), "merge")
        self._lin(self.merged[:nm], w["aligner.w1.weight"], self.h1[:nm])
        ck(k.ds41_vis_bias_act(lib.ptr(self.h1), lib.ptr(w["aligner.w1.bias"]), None, lib.ptr(self.h1), C.c_longlong(nm),
                               self.H, 1, st()), "gelu")
        self._lin(self.h1[:nm], w["aligner.w2.weight"], self.out[:nm])
        ck(k.ds41_vis_bias_act(lib.ptr(self.out), lib.ptr(w["aligner.w2.bias"]), None, lib.ptr(self.out),
                               C.c_longlong(nm), self.H, 0, st()), "bias")
        return self.out[:nm]

    def scatter(self, image_rows: torch.Tensor, row_ids: torch.Tensor, streams: torch.Tensor, copies: int = 4):
        """Write image rows into the residual streams [rows, copies, H] at `row_ids` (every stream copy gets the row)."""
        lib.check(lib.kernels().ds41_vis_scatter(lib.ptr(image_rows), lib.ptr(row_ids), lib.ptr(streams),
                                                 image_rows.shape[0], self.H, copies, lib.stream()), "scatter")
