"""Plain-PyTorch restatements of every quantisation format the engine uses.

These are the CPU oracles for the CUDA pack/unpack kernels and for the
block-scaled GEMMs.  Formats (reference: docs/ENGINEERING.md:27-33,
native/cuda/kernels/v41_kv.cu:15-46, native/include/ds41rt_v41_experts.h:55-62):

* FP8 E4M3 with fp32 scales per 1x128 (activations) / 128x128 (weights)  -- "f32 block" geometry
* FP8 E4M3 with UE8M0 scales per 32 elements (MX)                         -- official dense weights / window KV
* FP4 E2M1 with UE8M0 scales per 32 (MXFP4)                               -- official routed experts, index keys
* FP4 E2M1 with E4M3 scales per 16 and an fp32 global scale (NVFP4)       -- W4A4 variant, compressed KV
Two FP4 values share one byte; the even element is the low nibble.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
E2M1_MAX = 6.0
_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# midpoints between representable magnitudes and whether a tie rounds up (RNE on the code's LSB)
_E2M1_MID = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
_E2M1_TIE_UP = torch.tensor([False, True, False, True, False, True, False])


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Saturating round-to-nearest-even conversion to float8_e4m3fn."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 codes (uint8 in 0..15), saturating, round-nearest-even."""
    a = x.float().abs().clamp(max=E2M1_MAX)
    mid = _E2M1_MID.to(a.device)
    code = torch.bucketize(a, mid, right=False)         # a > mid -> next code; a == mid -> lower
    lower = (code - 0).clamp(max=6)
    tie = (a == mid[lower.clamp(max=6)]) & (code <= 6)
    tie_up = _E2M1_TIE_UP.to(a.device)[lower.clamp(max=6)]
    code = torch.where(tie & tie_up, code + 1, code).clamp(max=7)
    sign = (x < 0) | ((x == 0) & (torch.signbit(x.float())))
    return (code | (sign.to(torch.int64) << 3)).to(torch.uint8)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    vals = _E2M1_VALUES.to(code.device)
    mag = vals[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    """[..., n] codes -> [..., n/2] bytes, even element in the low nibble."""
    lo = codes[..., 0::2]
    hi = codes[..., 1::2]
    return (lo | (hi << 4)).to(torch.uint8)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = (packed >> 4) & 0xF
    return torch.stack([lo, hi], dim=-1).flatten(-2)


def ue8m0_ceil(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x (x > 0) as a biased exponent byte
    (native/cuda/kernels/v41_compressor.cu:28-40: exponent + (mantissa != 0))."""
    bits = x.float().clamp(min=2.0 ** -126).view(torch.int32)
    exp = (bits >> 23) & 0xFF
    exp = exp + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return exp.clamp(max=254).to(torch.uint8)


def ue8m0_to_float(e: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, e.float() - 127.0)


# ----------------------------------------------------------------------------- FP8, fp32 block scales
def quant_act_fp8_1x128(x: torch.Tensor, block: int = 128):
    """Per-row, per-`block` column group: scale = amax/448 (fp32); returns (e4m3, scales[rows, K/block])."""
    rows, k = x.shape
    assert k % block == 0
    g = x.float().view(rows, k // block, block)
    amax = g.abs().amax(-1).clamp(min=1e-10)
    scale = amax / E4M3_MAX
    q = to_e4m3(g / scale[..., None]).view(rows, k)
    return q, scale


def quant_weight_fp8_128x128(w: torch.Tensor, block: int = 128):
    n, k = w.shape
    nb, kb = (n + block - 1) // block, (k + block - 1) // block
    pad = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    pad[:n, :k] = w.float()
    g = pad.view(nb, block, kb, block)
    amax = g.abs().amax(dim=(1, 3)).clamp(min=1e-10)
    scale = amax / E4M3_MAX
    q = to_e4m3(g / scale[:, None, :, None]).view(nb * block, kb * block)[:n, :k].contiguous()
    return q, scale


def dequant_weight_fp8_128x128(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    n, k = q.shape
    s = scale.repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return q.float() * s


def dequant_act_fp8_1x128(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    return q.float() * scale.repeat_interleave(block, 1)[:, : q.shape[1]]


# ----------------------------------------------------------------------------- MX (UE8M0 per 32)
def quant_mxfp8(x: torch.Tensor, block: int = 32):
    """E4M3 payload + UE8M0 scale per `block` along the last dim; scale = ceil_pow2(amax/448)."""
    shape = x.shape
    g = x.float().reshape(-1, shape[-1] // block, block)
    amax = g.abs().amax(-1)
    e = ue8m0_ceil(amax / E4M3_MAX)
    q = to_e4m3(g / ue8m0_to_float(e)[..., None]).reshape(shape)
    return q, e.reshape(*shape[:-1], shape[-1] // block)


def dequant_mxfp8(q: torch.Tensor, e: torch.Tensor, block: int = 32) -> torch.Tensor:
    return q.float() * ue8m0_to_float(e).repeat_interleave(block, -1)


def qdq_mxfp8(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    q, e = quant_mxfp8(x, block)
    return dequant_mxfp8(q, e, block)


def quant_weight_mxfp8_32x32(w: torch.Tensor, block: int = 32):
    """Official dense-weight geometry: E4M3 + one UE8M0 scale per 32x32 tile."""
    n, k = w.shape
    assert n % block == 0 and k % block == 0
    g = w.float().view(n // block, block, k // block, block)
    amax = g.abs().amax(dim=(1, 3))
    e = ue8m0_ceil(amax / E4M3_MAX)
    q = to_e4m3(g / ue8m0_to_float(e)[:, None, :, None]).view(n, k)
    return q, e


def dequant_weight_mxfp8_32x32(q: torch.Tensor, e: torch.Tensor, block: int = 32) -> torch.Tensor:
    s = ue8m0_to_float(e).repeat_interleave(block, 0).repeat_interleave(block, 1)
    return q.float() * s


def quant_mxfp4(x: torch.Tensor, block: int = 32):
    """E2M1 codes packed two per byte + UE8M0 per `block`; scale = ceil_pow2(max(amax, 6*2^-126)/6)."""
    shape = x.shape
    g = x.float().reshape(-1, shape[-1] // block, block)
    amax = g.abs().amax(-1).clamp(min=E2M1_MAX * 2.0 ** -126)
    e = ue8m0_ceil(amax / E2M1_MAX)
    codes = e2m1_encode(g / ue8m0_to_float(e)[..., None]).reshape(shape)
    return pack_fp4(codes), e.reshape(*shape[:-1], shape[-1] // block)


def dequant_mxfp4(packed: torch.Tensor, e: torch.Tensor, block: int = 32) -> torch.Tensor:
    vals = e2m1_decode(unpack_fp4(packed))
    return vals * ue8m0_to_float(e).repeat_interleave(block, -1)


def qdq_mxfp4(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    p, e = quant_mxfp4(x, block)
    return dequant_mxfp4(p, e, block)


# ----------------------------------------------------------------------------- NVFP4 (E4M3 per 16 + global)
def quant_nvfp4(x: torch.Tensor, global_scale: torch.Tensor | float | None = None, block: int = 16):
    """Returns (packed, block_scales_e4m3, global_scale).  value = code * block_scale * global_scale.
    With global_scale None it is amax/(448*6), the ModelOpt convention."""
    shape = x.shape
    xf = x.float()
    if global_scale is None:
        global_scale = (xf.abs().amax().clamp(min=1e-12) / (E4M3_MAX * E2M1_MAX))
    gs = torch.as_tensor(global_scale, dtype=torch.float32, device=x.device)
    g = xf.reshape(-1, shape[-1] // block, block)
    amax = g.abs().amax(-1)
    bs = to_e4m3(amax / E2M1_MAX / gs)
    bsf = bs.float() * gs
    safe = torch.where(bsf == 0, torch.ones_like(bsf), bsf)
    codes = e2m1_encode(g / safe[..., None]).reshape(shape)
    return pack_fp4(codes), bs.reshape(*shape[:-1], shape[-1] // block), gs


def dequant_nvfp4(packed: torch.Tensor, bs: torch.Tensor, gs, block: int = 16) -> torch.Tensor:
    vals = e2m1_decode(unpack_fp4(packed))
    return vals * (bs.float() * gs).repeat_interleave(block, -1)


def quant_kv_fp4_e4m3_16(x: torch.Tensor):
    """Compressed-KV row format: E2M1 + E4M3 scale per 16, scale = e4m3(max(amax, 6*2^-9)/6)
    (native/cuda/kernels/v41_kv.cu:29-39)."""
    shape = x.shape
    g = x.float().reshape(-1, shape[-1] // 16, 16)
    amax = g.abs().amax(-1).clamp(min=E2M1_MAX * 2.0 ** -9)
    bs = to_e4m3(amax / E2M1_MAX)
    codes = e2m1_encode(g / bs.float()[..., None]).reshape(shape)
    return pack_fp4(codes), bs.reshape(*shape[:-1], shape[-1] // 16)


def dequant_kv_fp4_e4m3_16(packed: torch.Tensor, bs: torch.Tensor) -> torch.Tensor:
    return e2m1_decode(unpack_fp4(packed)) * bs.float().repeat_interleave(16, -1)


# ----------------------------------------------------------------------------- FP8 + UE8M0 block scales (128x128)
def quant_weight_fp8_ue8m0_block(w: torch.Tensor, block: int = 128):
    """E4M3 payload with one power-of-two scale per `block` x `block` tile (scale = ceil_pow2(amax/448)).
    Returns (q [n,k] float8, e [n/block, k/block] uint8)."""
    n, k = w.shape
    assert n % block == 0 and k % block == 0
    g = w.float().view(n // block, block, k // block, block)
    amax = g.abs().amax(dim=(1, 3))
    e = ue8m0_ceil(amax / E4M3_MAX)
    q = to_e4m3(g / ue8m0_to_float(e)[:, None, :, None]).view(n, k)
    return q, e


def expand_block_scales(e: torch.Tensor, block: int = 128, mx: int = 32) -> torch.Tensor:
    """[n/block, k/block] tile exponents -> per-row per-32 exponents [n, k/32] (what the MX GEMM consumes)."""
    return e.repeat_interleave(block, 0).repeat_interleave(block // mx, 1).contiguous()


def quant_act_fp8_ue8m0(x: torch.Tensor, group: int = 128):
    """Row-wise E4M3 payload with a power-of-two scale per `group` elements; exponents returned per 32."""
    q, e = quant_mxfp8(x, group)
    return q, e.repeat_interleave(group // 32, -1).contiguous()
