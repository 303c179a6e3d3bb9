// Elementwise and reduction kernels of the vision tower (ViT) and the aligner.  Every projection of the tower runs on
// the tcgen05 GEMM (gemm_tc.cu); attention is two batched GEMMs (Q K^T and P V per head over a query tile) around the
// row softmax below, so the only kernels here are the ones between GEMMs:
//   vis_rmsnorm     x [rows, W] bf16 -> bf16 (weight, eps)
//   vis_bias_act    y = act(x + bias) (+ residual), act 0 none / 1 GELU (erf)
//   vis_silu_mul    [rows, 2I] (gate | up) -> [rows, I]
//   vis_rope2d      rotate q and k inside a [rows, 3W] qkv buffer: the first half of every head by the patch row,
//                   the second half by the patch column (pairs (2i, 2i+1), theta^(-2i/(d/2)))
//   vis_softmax     fp32 scores [rows, n] (ld) -> bf16 probabilities, with scale; columns >= n_valid masked
//   vis_merge       [gh*gw, W] patch grid -> [gh/m * gw/m, m*m*W] (m x m neighbourhoods concatenated, row-major inside)
//   vis_scatter     copy rows into the embedding stream at given row indices (image token positions)
// Reference: native/cuda/kernels/v41_vision.cu:32-117 (elementwise ops), :151,196-208 (projection / attention GEMMs).
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

__global__ void __launch_bounds__(256)
vis_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ out, int W, float eps) {
  __shared__ float part[8];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* xr = x + 1ll * r * W;
  float sq = 0.f;
  for (int c = tid * 2; c < W; c += 512) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    sq = fmaf(v.x, v.x, fmaf(v.y, v.y, sq));
  }
  sq = warp_sum(sq);
  if ((tid & 31) == 0) part[tid >> 5] = sq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += part[i];
  const float inv = rsqrtf(tot / W + eps);
  for (int c = tid * 2; c < W; c += 512) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + c));
    *reinterpret_cast<__nv_bfloat162*>(out + 1ll * r * W + c) = __floats2bfloat162_rn(v.x * inv * g.x, v.y * inv * g.y);
  }
}

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); }

__global__ void __launch_bounds__(256)
vis_bias_act_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ bias,
                    const __nv_bfloat16* residual, __nv_bfloat16* out, long long n, int cols,
                    int act) {
  // x or residual may be the output buffer (in-place calls): no __restrict__, so they are read with coherent loads
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (1ll * blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= n) return;
  const int c = static_cast<int>(i % cols);
  float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + i));
  if (bias != nullptr) {
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bias + c));
    v.x += b.x;
    v.y += b.y;
  }
  if (act == 1) {
    v.x = gelu_erf(v.x);
    v.y = gelu_erf(v.y);
  }
  if (residual != nullptr) {
    const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(residual + i));
    v.x += r.x;
    v.y += r.y;
  }
  *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(v.x, v.y);
}

__global__ void __launch_bounds__(256)
vis_silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (1ll * blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= 1ll * rows * I) return;
  const long long r = i / I;
  const int c = static_cast<int>(i - r * I);
  const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * I + c));
  const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * I + I + c));
  *reinterpret_cast<__nv_bfloat162*>(out + i) =
      __floats2bfloat162_rn(g.x / (1.0f + __expf(-g.x)) * u.x, g.y / (1.0f + __expf(-g.y)) * u.y);
}

// one block per patch row; thread t handles pair t of every head of q and k
__global__ void __launch_bounds__(256)
vis_rope2d_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos_hw, int W, int heads, float theta) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int d = W / heads, half = d / 2;            // half of the head dim per axis
  const int ph = pos_hw[2 * r], pw = pos_hw[2 * r + 1];
  for (int idx = threadIdx.x; idx < heads * (d / 2); idx += blockDim.x) {
    const int h = idx / (d / 2), pair = idx % (d / 2);
    const int e = 2 * pair;                          // element offset inside the head
    const bool second = e >= half;
    const int i = (second ? e - half : e) / 2;       // frequency index within the axis
    const float freq = powf(theta, -2.0f * i / half);
    const float ang = (second ? pw : ph) * freq;
    float sn, cs;
    sincosf(ang, &sn, &cs);
#pragma unroll
    for (int which = 0; which < 2; ++which) {        // q then k
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(qkv + 1ll * r * 3 * W + which * W + h * d + e);
      const float2 v = __bfloat1622float2(*p);
      *p = __floats2bfloat162_rn(v.x * cs - v.y * sn, v.y * cs + v.x * sn);
    }
  }
}

__global__ void __launch_bounds__(256)
vis_softmax_kernel(const float* __restrict__ s, long long ld, int n_valid, float scale, __nv_bfloat16* __restrict__ p,
                   long long ldp, int n_pad) {
  __shared__ float part[8];
  __shared__ float bcast;
  pdl_launch_dependents();
  pdl_wait();
  const long long r = blockIdx.x;
  const int tid = threadIdx.x;
  const float* row = s + r * ld;
  float m = -INFINITY;
  for (int c = tid; c < n_valid; c += 256) m = fmaxf(m, row[c] * scale);
  m = warp_max(m);
  if ((tid & 31) == 0) part[tid >> 5] = m;
  __syncthreads();
  if (tid == 0) {
    float t = part[0];
    for (int i = 1; i < 8; ++i) t = fmaxf(t, part[i]);
    bcast = t;
  }
  __syncthreads();
  m = bcast;
  float sum = 0.f;
  for (int c = tid; c < n_valid; c += 256) sum += __expf(row[c] * scale - m);
  sum = warp_sum(sum);
  __syncthreads();
  if ((tid & 31) == 0) part[tid >> 5] = sum;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += part[i];
    bcast = 1.0f / t;
  }
  __syncthreads();
  const float inv = bcast;
  for (int c = tid; c < n_pad; c += 256)
    p[r * ldp + c] = __float2bfloat16_rn(c < n_valid ? __expf(row[c] * scale - m) * inv : 0.f);
}

__global__ void __launch_bounds__(256)
vis_merge_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int gh, int gw, int m, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int o = blockIdx.x;                          // merged token
  const int ow = gw / m;
  const int oy = o / ow, ox = o % ow;
  const int vec = W / 8;
  for (int idx = threadIdx.x; idx < m * m * vec; idx += blockDim.x) {
    const int cell = idx / vec, v = idx % vec;
    const int sy = oy * m + cell / m, sx = ox * m + cell % m;
    *reinterpret_cast<uint4*>(out + (1ll * o * m * m + cell) * W + v * 8) =
        *reinterpret_cast<const uint4*>(x + (1ll * sy * gw + sx) * W + v * 8);
  }
}

__global__ void __launch_bounds__(256)
vis_scatter_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ rows, __nv_bfloat16* __restrict__ dst,
                   int H, int copies) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows[i];
  if (r < 0) return;
  for (int idx = threadIdx.x; idx < copies * (H / 8); idx += blockDim.x) {
    const int cp = idx / (H / 8), v = idx % (H / 8);
    *reinterpret_cast<uint4*>(dst + (1ll * r * copies + cp) * H + v * 8) =
        *reinterpret_cast<const uint4*>(src + 1ll * i * H + v * 8);
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_vis_rmsnorm(const void* x, const void* w, void* out, int rows, int W, float eps, void* stream) {
  if (rows <= 0 || W <= 0 || (W & 1)) return cudaErrorInvalidValue;
  return launch_pdl(vis_rmsnorm_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                    static_cast<__nv_bfloat16*>(out), W, eps);
}

extern "C" int ds41_vis_bias_act(const void* x, const void* bias, const void* residual, void* out, long long rows,
                                 int cols, int act, void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 1) || act < 0 || act > 1) return cudaErrorInvalidValue;
  const long long n = rows * cols;
  return launch_pdl(vis_bias_act_kernel, dim3(static_cast<unsigned>((n / 2 + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x),
                    static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual),
                    static_cast<__nv_bfloat16*>(out), n, cols, act);
}

extern "C" int ds41_vis_silu_mul(const void* gu, void* out, int rows, int I, void* stream) {
  if (rows <= 0 || I <= 0 || (I & 1)) return cudaErrorInvalidValue;
  const long long n = 1ll * rows * I;
  return launch_pdl(vis_silu_mul_kernel, dim3(static_cast<unsigned>((n / 2 + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(gu),
                    static_cast<__nv_bfloat16*>(out), rows, I);
}

extern "C" int ds41_vis_rope2d(void* qkv, const int* pos_hw, int rows, int W, int heads, float theta, void* stream) {
  if (rows <= 0 || heads <= 0 || W % heads != 0 || ((W / heads) & 3)) return cudaErrorInvalidValue;
  return launch_pdl(vis_rope2d_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<__nv_bfloat16*>(qkv), pos_hw, W, heads, theta);
}

extern "C" int ds41_vis_softmax(const float* s, long long ld, long long rows, int n_valid, float scale, void* p,
                                long long ldp, int n_pad, void* stream) {
  if (rows <= 0 || n_valid <= 0 || n_pad < n_valid) return cudaErrorInvalidValue;
  return launch_pdl(vis_softmax_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), s, ld, n_valid, scale, static_cast<__nv_bfloat16*>(p), ldp, n_pad);
}

extern "C" int ds41_vis_merge(const void* x, void* out, int gh, int gw, int m, int W, void* stream) {
  if (gh <= 0 || gw <= 0 || m <= 0 || gh % m || gw % m || (W & 7)) return cudaErrorInvalidValue;
  return launch_pdl(vis_merge_kernel, dim3((gh / m) * (gw / m)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), gh, gw, m, W);
}

extern "C" int ds41_vis_scatter(const void* src, const int* rows, void* dst, int n, int H, int copies, void* stream) {
  if (n <= 0 || (H & 7) || copies <= 0) return cudaErrorInvalidValue;
  return launch_pdl(vis_scatter_kernel, dim3(n), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(src), rows, static_cast<__nv_bfloat16*>(dst), H, copies);
}
