// Activation quantisation for the block-scaled tensor-core GEMMs.
//
//  act_quant_mx : bf16 [batch][rows][K] -> E4M3 payload + UE8M0 scales written directly in the 512-byte
//                 scale-factor atom layout the MX GEMM copies into TMEM
//                 (byte = (row%32)*16 + ((row/32)%4)*4 + kblock%4, atoms [row/128][K/128]).
//                 `group` = 32 gives one scale per 32 elements (MX); `group` = 128 gives the 1x128
//                 activation-scale geometry (the same exponent is written to the four 32-blocks).
//                 scale = smallest power of two >= amax/448  (quantise contract of the reference's
//                 native/include/ds41rt_v41_experts.h:55-62 and native/cuda/kernels/v41_kv.cu:15-46).
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

static int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

struct ActQuantParams {
  const __nv_bfloat16* x;
  long long ldx, x_batch_stride;
  uint8_t* q;
  long long ldq, q_batch_stride;
  uint8_t* sf;
  long long sf_batch_stride;
  int rows, K, batch, group;
  const int* n_active;
};

// one warp per (row, 128-wide K chunk); 8 warps per block
__global__ void __launch_bounds__(256) act_quant_mx_kernel(ActQuantParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunks = p.K / 128;
  const long long item = 1ll * blockIdx.x * 8 + warp;
  const int b = blockIdx.y;
  pdl_launch_dependents();
  pdl_wait();
  if (p.n_active != nullptr && b >= *p.n_active) return;
  if (item >= 1ll * p.rows * chunks) return;
  const int r = static_cast<int>(item / chunks), kc = static_cast<int>(item % chunks);
  const __nv_bfloat16* src = p.x + b * p.x_batch_stride + 1ll * r * p.ldx + kc * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y)));
  // 8 lanes share a 32-element block
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  if (p.group == 128) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
  }
  const uint32_t e = ue8m0_ceil_exp(amax * (1.0f / 448.0f));
  const float inv = __uint_as_float((254u - e) << 23);          // 2^-(e-127)
  const __nv_fp8x4_e4m3 packed(make_float4(a.x * inv, a.y * inv, c.x * inv, c.y * inv));
  *reinterpret_cast<uint32_t*>(p.q + b * p.q_batch_stride + 1ll * r * p.ldq + kc * 128 + lane * 4) =
      *reinterpret_cast<const uint32_t*>(&packed);
  if ((lane & 7) == 0) {
    const int kb = lane >> 3;
    uint8_t* atom = p.sf + b * p.sf_batch_stride + (1ll * (r / 128) * chunks + kc) * 512;
    atom[(r % 32) * 16 + ((r / 32) % 4) * 4 + kb] = static_cast<uint8_t>(e);
  }
}

// Prefill-sized variant (1x128 scales): one warp per row, 16 bytes per lane, two 128-wide K chunks per step; only rows
// below *rows_dev (a device count, e.g. the rows an expert-parallel rank received) are touched.
__global__ void __launch_bounds__(256)
act_quant_mx_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                         uint8_t* __restrict__ sf, int rows, int K, const int* __restrict__ rows_dev) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int live = rows_dev != nullptr ? min(rows, *rows_dev) : rows;
  const int chunks = K / 128;
  for (int r = blockIdx.x * 8 + warp; r < live; r += gridDim.x * 8) {
    const __nv_bfloat16* src = x + 1ll * r * ldx;
    uint8_t* dst = q + 1ll * r * ldq;
    uint8_t* atom_row = sf + 1ll * (r / 128) * chunks * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += 256) {
      const int k = k0 + lane * 8;
      float f[8];
      float amax = 0.f;
      if (k < K) {
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
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
      if (k < K) {
        const uint32_t e = ue8m0_ceil_exp(amax * (1.0f / 448.0f));
        const float inv = __uint_as_float((254u - e) << 23);
        const __nv_fp8x4_e4m3 lo(make_float4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv));
        const __nv_fp8x4_e4m3 hi(make_float4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst + k) = o;
        if ((lane & 15) == 0)
          *reinterpret_cast<uint32_t*>(atom_row + 1ll * (k / 128) * 512) = e * 0x01010101u;
      }
    }
  }
}

// NVFP4 activation rows: e2m1 values (two per byte, even element in the low nibble) with one E4M3 scale per 16
// elements, relative to a fixed per-tensor scale `global_scale` (value = code * block_scale * global_scale).
// block_scale = e4m3(amax / 6 / global_scale); codes round to nearest (ties to even) on the e2m1 grid.
// One warp per row, 8 elements per lane per step (two lanes share a 16-element block).  Scales go straight into the
// 512-byte atoms of the tensor-core kind: atom [row/128][k/64], byte (row%32)*16 + ((row/32)%4)*4 + (k/16)%4.
__global__ void __launch_bounds__(256)
act_quant_nvfp4_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                            uint8_t* __restrict__ sf, int rows, int K, float global_scale,
                            const int* __restrict__ rows_dev, long long x_bs, long long q_bs, long long sf_bs,
                            const int* __restrict__ n_active) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  if (n_active != nullptr && b >= *n_active) return;
  const int live = rows_dev != nullptr ? min(rows, *rows_dev) : rows;
  const int k_atoms = K / 64;
  x += b * x_bs;
  q += b * (q_bs / 2);
  sf += b * sf_bs;
  for (int r = blockIdx.x * 8 + warp; r < live; r += gridDim.x * 8) {
    const __nv_bfloat16* src = x + 1ll * r * ldx;
    uint8_t* dst = q + 1ll * r * (ldq / 2);
    uint8_t* atom_row = sf + 1ll * (r / 128) * k_atoms * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += 256) {
      const int k = k0 + lane * 8;
      float f[8];
      float amax = 0.f;
      if (k < K) {
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
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));       // 16-element block = two lanes
      if (k < K) {
        // IEEE divisions in this order, so that scales and codes are bit-identical to the host oracle
        const __nv_fp8_e4m3 bs(__fdiv_rn(__fdiv_rn(amax, 6.0f), global_scale));
        const float bsf = __fmul_rn(static_cast<float>(bs), global_scale);
        const float den = bsf == 0.f ? 1.0f : bsf;
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) packed |= e2m1_code(__fdiv_rn(f[j], den)) << (4 * j);
        *reinterpret_cast<uint32_t*>(dst + k / 2) = packed;
        if ((lane & 1) == 0) atom_row[1ll * (k / 64) * 512 + ((k / 16) & 3)] = bs.__x;
      }
    }
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_act_quant_nvfp4_rows(const void* x, long long ldx, void* q, long long ldq, void* sf, int rows,
                                         int K, float global_scale, const int* rows_dev, int batch,
                                         long long x_batch_stride, long long q_batch_stride, long long sf_batch_stride,
                                         const int* n_active, void* stream) {
  if (rows <= 0 || K <= 0 || K % 64 != 0 || (ldx & 7) || (ldq & 7) || !(global_scale > 0.f) || batch <= 0 ||
      (q_batch_stride & 1))
    return cudaErrorInvalidValue;
  const int blocks = min((rows + 7) / 8, 8 * sm_count_cached());
  return launch_pdl(act_quant_nvfp4_rows_kernel, dim3(blocks, batch), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(sf),
                    rows, K, global_scale, rows_dev, x_batch_stride, q_batch_stride, sf_batch_stride, n_active);
}

extern "C" int ds41_act_quant_mx_rows(const void* x, long long ldx, void* q, long long ldq, void* sf, int rows, int K,
                                      const int* rows_dev, void* stream) {
  if (rows <= 0 || K <= 0 || K % 128 != 0 || (ldx & 7) || (ldq & 7)) return cudaErrorInvalidValue;
  const int blocks = min((rows + 7) / 8, 8 * sm_count_cached());
  return launch_pdl(act_quant_mx_rows_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(sf),
                    rows, K, rows_dev);
}

extern "C" int ds41_act_quant_mx(const void* x, long long ldx, long long x_batch_stride, void* q, long long ldq,
                                 long long q_batch_stride, void* sf, long long sf_batch_stride, int rows, int K,
                                 int batch, int group, const int* n_active, void* stream) {
  if (rows <= 0 || K <= 0 || K % 128 != 0 || batch <= 0 || (group != 32 && group != 128) || (ldx & 3) || (ldq & 3))
    return cudaErrorInvalidValue;
  ActQuantParams p{static_cast<const __nv_bfloat16*>(x), ldx, x_batch_stride, static_cast<uint8_t*>(q), ldq,
                   q_batch_stride, static_cast<uint8_t*>(sf), sf_batch_stride, rows, K, batch, group, n_active};
  const long long items = 1ll * rows * (K / 128);
  dim3 grid(static_cast<unsigned>((items + 7) / 8), batch);
  return launch_pdl(act_quant_mx_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}
