// Engram memory on the GPU: row dequantisation and the gated residual update.
//
//  engram_dequant : hashed table rows as stored (256 e4m3 values + 8 UE8M0 scales, one per 32 values) -> bf16
//  engram_dequant_nvfp4 : rows of a converted table (128 bytes of E2M1 pairs, even element in the low nibble, + 16
//                   E4M3 scales, one per 16 values; one fp32 scale per table) -> bf16((code * scale) * table scale)
//  engram_gate    : for every token row and residual stream s (4 streams):
//                     dot  = sum_c x[s,c] * (q_w[s,c] * k_w[s,c]) * key[s,c]
//                     dot *= rsqrt(mean x^2 + eps) * rsqrt(mean key^2 + eps) / sqrt(H)
//                     gate = sigmoid(sign(dot) * sqrt(max(|dot|, 1e-6)))
//                     out[s,:] = x[s,:] + gate * value[:]
//                   kv holds 4 keys and then 1 value of H columns per row (the output of the engram.wkv projection);
//                   rows whose text_mask byte is 0 (image positions) pass through unchanged.
// One block per token row: the four streams are handled by two warps each, rows are read with 16-byte loads and
// the value vector is read once for all four streams.
// Behaviour reference: native/cuda/kernels/engram.cu:19-71 (gate) and :88-110 (row dequant) of the reference.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

__global__ void __launch_bounds__(256)
engram_dequant_kernel(const uint8_t* __restrict__ rows_q, int row_bytes, int dim, __nv_bfloat16* __restrict__ out,
                      int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  // one warp per row: 8 values per lane per step
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_rows) return;
  const uint8_t* src = rows_q + 1ll * warp * row_bytes;
  for (int c = lane * 8; c < dim; c += 256) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + c);
    const uint32_t e = src[dim + (c >> 5)];
    // exponent 255 encodes NaN, exponent 0 is 2^-127 (a subnormal float)
    const float sc = e == 255 ? __int_as_float(0x7fc00000) : __uint_as_float(e == 0 ? 0x00400000u : e << 23);
    const __nv_fp8x2_storage_t* q2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(q2[q], __NV_E4M3)));
      o2[q] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
    *reinterpret_cast<uint4*>(out + 1ll * warp * dim + c) = o;
  }
}

__global__ void __launch_bounds__(256)
engram_dequant_nvfp4_kernel(const uint8_t* __restrict__ rows_q, int row_bytes, int dim, float table_scale,
                            __nv_bfloat16* __restrict__ out, int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  // one warp per row: 8 values (4 payload bytes, half a scale group) per lane per step
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_rows) return;
  const uint8_t* src = rows_q + 1ll * warp * row_bytes;
  for (int c = lane * 8; c < dim; c += 256) {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(src + (c >> 1));
    __nv_fp8_e4m3 s8;
    s8.__x = src[(dim >> 1) + (c >> 4)];
    const float sc = static_cast<float>(s8);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_fp4x2_storage_t pair = static_cast<__nv_fp4x2_storage_t>((raw >> (8 * q)) & 0xffu);
      const float2 f = __half22float2(__half2(__nv_cvt_fp4x2_to_halfraw2(pair, __NV_E2M1)));
      o2[q] = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(f.x, sc), table_scale), __fmul_rn(__fmul_rn(f.y, sc), table_scale));
    }
    *reinterpret_cast<uint4*>(out + 1ll * warp * dim + c) = o;
  }
}

__global__ void __launch_bounds__(256)
engram_gate_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ kv,
                   const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w,
                   const uint8_t* __restrict__ text_mask, __nv_bfloat16* out, int H, float eps) {
  // x and out are the same buffer in the engine (streams updated in place): they are not declared __restrict__, so
  // that x is read with ordinary coherent loads.  A read-only-path load would leave lines in this SM's cache that the
  // stores below do not refresh, and a dependent kernel that was launched early (its cache flush already done) could
  // read those stale lines.
  __shared__ float part[3][8];
  __shared__ float gate_s[4];
  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s = warp >> 1;                     // stream of this warp pair
  const int half = warp & 1;
  pdl_launch_dependents();
  pdl_wait();
  const __nv_bfloat16* xs = x + (1ll * row * 4 + s) * H;
  __nv_bfloat16* os = out + (1ll * row * 4 + s) * H;
  if (text_mask != nullptr && text_mask[row] == 0) {
    for (int c = (half * 32 + lane) * 8; c < H; c += 512) *reinterpret_cast<uint4*>(os + c) = *reinterpret_cast<const uint4*>(xs + c);
    return;
  }
  const __nv_bfloat16* key = kv + (1ll * row * 5 + s) * H;
  const __nv_bfloat16* val = kv + (1ll * row * 5 + 4) * H;
  float xx = 0.f, kk = 0.f, dot = 0.f;
  for (int c = (half * 32 + lane) * 8; c < H; c += 512) {
    const uint4 xr = *reinterpret_cast<const uint4*>(xs + c);
    const uint4 kr = *reinterpret_cast<const uint4*>(key + c);
    const uint4 qr = *reinterpret_cast<const uint4*>(q_w + 1ll * s * H + c);
    const uint4 wr = *reinterpret_cast<const uint4*>(k_w + 1ll * s * H + c);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xr);
    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kr);
    const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qr);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xv = __bfloat1622float2(x2[j]), kv2 = __bfloat1622float2(k2[j]);
      const float2 qv = __bfloat1622float2(q2[j]), wv = __bfloat1622float2(w2[j]);
      xx = fmaf(xv.x, xv.x, fmaf(xv.y, xv.y, xx));
      kk = fmaf(kv2.x, kv2.x, fmaf(kv2.y, kv2.y, kk));
      dot = fmaf(xv.x * (qv.x * wv.x), kv2.x, fmaf(xv.y * (qv.y * wv.y), kv2.y, dot));
    }
  }
  xx = warp_sum(xx);
  kk = warp_sum(kk);
  dot = warp_sum(dot);
  if (lane == 0) {
    part[0][warp] = xx;
    part[1][warp] = kk;
    part[2][warp] = dot;
  }
  __syncthreads();
  if (tid < 4) {
    const float sx = part[0][2 * tid] + part[0][2 * tid + 1];
    const float sk = part[1][2 * tid] + part[1][2 * tid + 1];
    float d = part[2][2 * tid] + part[2][2 * tid + 1];
    d = d * rsqrtf(sx / H + eps) * rsqrtf(sk / H + eps) * rsqrtf(static_cast<float>(H));
    const float t = copysignf(sqrtf(fmaxf(fabsf(d), 1e-6f)), d);
    gate_s[tid] = 1.0f / (1.0f + __expf(-t));
  }
  __syncthreads();
  const float g = gate_s[s];
  for (int c = (half * 32 + lane) * 8; c < H; c += 512) {
    const uint4 xr = *reinterpret_cast<const uint4*>(xs + c);
    const uint4 vr = *reinterpret_cast<const uint4*>(val + c);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xr);
    const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vr);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xv = __bfloat1622float2(x2[j]), vv = __bfloat1622float2(v2[j]);
      o2[j] = __floats2bfloat162_rn(fmaf(g, vv.x, xv.x), fmaf(g, vv.y, xv.y));
    }
    *reinterpret_cast<uint4*>(os + c) = o;
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_engram_dequant(const void* rows_q, int row_bytes, int dim, void* out, int n_rows, void* stream) {
  if (rows_q == nullptr || out == nullptr || n_rows <= 0 || dim <= 0 || (dim & 31) || row_bytes < dim + dim / 32 ||
      (row_bytes & 7))
    return cudaErrorInvalidValue;
  const int blocks = (n_rows + 7) / 8;
  return launch_pdl(engram_dequant_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint8_t*>(rows_q), row_bytes, dim, static_cast<__nv_bfloat16*>(out), n_rows);
}

extern "C" int ds41_engram_dequant_nvfp4(const void* rows_q, int row_bytes, int dim, float table_scale, void* out,
                                         int n_rows, void* stream) {
  if (rows_q == nullptr || out == nullptr || n_rows <= 0 || dim <= 0 || (dim & 31) ||
      row_bytes < dim / 2 + dim / 16 || (row_bytes & 3) || !(table_scale > 0.0f) || !isfinite(table_scale))
    return cudaErrorInvalidValue;
  const int blocks = (n_rows + 7) / 8;
  return launch_pdl(engram_dequant_nvfp4_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint8_t*>(rows_q), row_bytes, dim, table_scale,
                    static_cast<__nv_bfloat16*>(out), n_rows);
}

extern "C" int ds41_engram_gate(const void* x, const void* kv, const void* q_w, const void* k_w,
                                const uint8_t* text_mask, void* out, int rows, int H, float eps, void* stream) {
  if (x == nullptr || kv == nullptr || q_w == nullptr || k_w == nullptr || out == nullptr || rows <= 0 || H <= 0 ||
      (H & 7))
    return cudaErrorInvalidValue;
  return launch_pdl(engram_gate_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(kv),
                    static_cast<const __nv_bfloat16*>(q_w), static_cast<const __nv_bfloat16*>(k_w), text_mask,
                    static_cast<__nv_bfloat16*>(out), H, eps);
}
