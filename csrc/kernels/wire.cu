// Hidden-state rows on the wire: one record per row of H E4M3 values followed by H/32 UE8M0 scales (5280 bytes for
// H = 5120, a 1.94x smaller record than bf16), for hand-offs whose cost is the link and not the arithmetic.
//
//   wire_encode : bf16 [rows, H] -> records; scale of a group of 32 = smallest power of two >= amax / 448
//   wire_decode : records -> bf16(value * scale)   (exponent byte 255 decodes to NaN, 0 to 2^-127)
// One warp per row, 8 values per lane per step; a group of 32 is four neighbouring lanes.
// Decode arithmetic follows the reference's row decoder for the same record (native/cuda/kernels/v41_exl3_wire.cu:9-18
// of the reference); the encoder is the counterpart the reference runs on its worker side.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"
#include "ds41_tma.h"

namespace ds41 {

__global__ void __launch_bounds__(256)
wire_encode_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ out, long long row_bytes,
                   int rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += (gridDim.x * blockDim.x) >> 5) {
    const __nv_bfloat16* src = x + 1ll * r * ldx;
    uint8_t* dst = out + 1ll * r * row_bytes;
    for (int k0 = 0; k0 < H; k0 += 256) {
      const int k = k0 + lane * 8;
      float f[8];
      float amax = 0.f;
      if (k < H) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + k);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 v = __bfloat1622float2(h[j]);
          f[2 * j] = v.x;
          f[2 * j + 1] = v.y;
          amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
        }
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      if (k < H) {
        const uint32_t e = ue8m0_ceil_exp(amax * (1.0f / 448.0f));
        const float inv = __uint_as_float((254u - e) << 23);
        const __nv_fp8x4_e4m3 lo(make_float4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv));
        const __nv_fp8x4_e4m3 hi(make_float4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst + k) = o;
        if ((lane & 3) == 0) dst[H + (k >> 5)] = static_cast<uint8_t>(e);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
wire_decode_kernel(const uint8_t* __restrict__ in, long long row_bytes, __nv_bfloat16* __restrict__ y, long long ldy,
                   int rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += (gridDim.x * blockDim.x) >> 5) {
    const uint8_t* src = in + 1ll * r * row_bytes;
    __nv_bfloat16* dst = y + 1ll * r * ldy;
    for (int k = lane * 8; k < H; k += 256) {
      const uint2 raw = *reinterpret_cast<const uint2*>(src + k);
      const uint32_t e = src[H + (k >> 5)];
      const float sc = e == 255 ? __int_as_float(0x7fc00000) : __uint_as_float(e == 0 ? 0x00400000u : e << 23);
      const __nv_fp8x2_storage_t* q2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(q2[q], __NV_E4M3)));
        o2[q] = __floats2bfloat162_rn(__fmul_rn(f.x, sc), __fmul_rn(f.y, sc));
      }
      *reinterpret_cast<uint4*>(dst + k) = o;
    }
  }
}

}  // namespace ds41

using namespace ds41;

static bool wire_geometry_ok(const void* a, const void* b, int rows, int H, long long ld, long long row_bytes) {
  return a != nullptr && b != nullptr && rows > 0 && H > 0 && (H & 31) == 0 && (ld & 7) == 0 && ld >= H &&
         row_bytes >= H + H / 32 && (row_bytes & 7) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(b) & 15) == 0;
}

extern "C" int ds41_wire_encode(const void* x, long long ldx, void* out, long long row_bytes, int rows, int H,
                                void* stream) {
  if (!wire_geometry_ok(x, out, rows, H, ldx, row_bytes)) return cudaErrorInvalidValue;
  const int blocks = min((rows + 7) / 8, 8 * sm_count());
  return launch_pdl(wire_encode_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(out), row_bytes, rows, H);
}

extern "C" int ds41_wire_decode(const void* in, long long row_bytes, void* y, long long ldy, int rows, int H,
                                void* stream) {
  if (!wire_geometry_ok(in, y, rows, H, ldy, row_bytes)) return cudaErrorInvalidValue;
  const int blocks = min((rows + 7) / 8, 8 * sm_count());
  return launch_pdl(wire_decode_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint8_t*>(in), row_bytes, static_cast<__nv_bfloat16*>(y), ldy, rows, H);
}
