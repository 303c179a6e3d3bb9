// Fused hyper-connection step for small row counts (decode / verification chunks): ONE launch closes a
// sublayer and opens the next one.
//
//   grid (H / 128, rows).  Block (slice, row):
//     1. expand     streams'[d] = post[d]*sub + sum_s comb[s][d]*streams[s] for its 128 columns, where `sub` is the
//                   sum of the sublayer's fp32 partial planes (this GPU's split-K planes and every peer's planes,
//                   read over NVLink after a bounded wait on the peers' epoch flags);
//     2. collapse   because the collapse weights of the sublayer being opened are already known (they come from
//                   the PREVIOUS mixes), the block also writes x = sum_d pre[d]*streams'[d] for its columns and
//                   their sum of squares;
//     3. mixes      its share of the 24 projections of the NEXT mixes (and of the streams' sum of squares).
//   The block that arrives last for its row (ticket counter, released with __threadfence) reduces the slice
//   partials in a fixed order, derives next_pre / post / comb (Sinkhorn in warp 0) and RMS-normalises the
//   collapsed row into bf16 (optionally also into E4M3 + scale atoms for the block-scaled expert GEMM).
//
// Mathematics: native/cuda/kernels/v41_hc.cu:6-29,70-120 and rust/crates/ds41rt-daemon/src/v41_hc.rs:153-225 of the
// reference; the fusion and the one-shot cross-rank sum are this design's.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

constexpr int kMult = 4;
constexpr int kProj = 2 * kMult + kMult * kMult;   // 24
constexpr int kSlice = 128;
constexpr int kStride = kProj + 2;                 // 24 dots, sum sq streams, sum sq collapsed

struct StepParts {
  const float* base[8];
  int n_ranks, n_splits;
  long long split_stride;
};

struct HcStepParams {
  const __nv_bfloat16* streams_in;
  __nv_bfloat16* streams_out;
  StepParts parts;
  const float* post;        // coefficients of the sublayer being closed
  const float* comb;
  const float* pre_in;      // collapse weights of the sublayer being opened
  const float* fn;          // next mixes: [24][4H], scale[3], base[24]
  const float* scale;
  const float* base;
  const float* norm_w;
  float* partial;           // [slices][rows][26]
  float* xc;                // [rows][H] collapsed, un-normalised
  float* next_pre;
  float* post_out;
  float* comb_out;
  __nv_bfloat16* xn;
  float* tap_mean;
  uint8_t* xq;
  uint8_t* xq_sf;
  unsigned int* tickets;    // [rows]; zero before the first launch, reset by the finishing block
  int rows, H, iters;
  float hc_eps, norm_eps;
  const uint32_t* const* wait_flags;
  const uint32_t* wait_epoch;
  int* status;
};

__global__ void __launch_bounds__(256) hc_step_kernel(HcStepParams p) {
  __shared__ float xs[kMult][kSlice];
  __shared__ float sqc[kSlice];
  __shared__ float proj[kStride];
  __shared__ int s_last;
  const int c0 = blockIdx.x * kSlice, r = blockIdx.y, H = p.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_slices = gridDim.x;
  pdl_launch_dependents();
  pdl_wait();
  if (p.wait_flags != nullptr && p.parts.n_ranks > 1) {
    if (tid < p.parts.n_ranks) flag_wait_ge(p.wait_flags[tid], *p.wait_epoch, p.status, 400 + tid);
    __syncthreads();
  }
  float* my_partial = p.partial + (1ll * blockIdx.x * p.rows + r) * kStride;
  // ---------------------------------------------------------------- 1+2: expand and collapse one column per thread
  if (tid < kSlice) {
    const int c = c0 + tid;
    float s_in[kMult], out[kMult];
#pragma unroll
    for (int s = 0; s < kMult; ++s) s_in[s] = __bfloat162float(p.streams_in[(1ll * r * kMult + s) * H + c]);
    if (p.parts.n_ranks > 0) {
      // Partial planes of every rank, summed in rank-major, split-minor order.  The loads of 32 planes are issued
      // before the first add: a load from a peer takes a few microseconds, and one at a time they were most of this
      // kernel's time on 8 GPUs.
      float sub = 0.f;
      const int n_sp = p.parts.n_splits, total = p.parts.n_ranks * n_sp;
      for (int j0 = 0; j0 < total; j0 += 32) {
        float v[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const int j = j0 + u;
          v[u] = 0.f;
          if (j < total) {
            const int k = j / n_sp, sp = j - k * n_sp;
            v[u] = p.parts.base[k][1ll * r * H + c + sp * p.parts.split_stride];
          }
        }
#pragma unroll
        for (int u = 0; u < 32; ++u) sub += v[u];
      }
      sub = bf16_round(sub);
#pragma unroll
      for (int d = 0; d < kMult; ++d) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < kMult; ++s) acc = fmaf(p.comb[r * 16 + s * 4 + d], s_in[s], acc);
        out[d] = bf16_round(fmaf(p.post[r * 4 + d], sub, acc));
        p.streams_out[(1ll * r * kMult + d) * H + c] = __float2bfloat16_rn(out[d]);
      }
    } else {
#pragma unroll
      for (int d = 0; d < kMult; ++d) out[d] = s_in[d];
    }
    float col = 0.f, mean = 0.f;
#pragma unroll
    for (int d = 0; d < kMult; ++d) {
      xs[d][tid] = out[d];
      col = fmaf(p.pre_in[r * 4 + d], out[d], col);
      mean += out[d];
    }
    col = bf16_round(col);
    p.xc[1ll * r * H + c] = col;
    sqc[tid] = col * col;
    if (p.tap_mean != nullptr) p.tap_mean[1ll * r * H + c] = 0.25f * mean;
  }
  __syncthreads();
  // ---------------------------------------------------------------- 3: slice share of the next mixes
  {
    float dot[3] = {0.f, 0.f, 0.f};
    float sq = 0.f;
#pragma unroll 8
    for (int idx = lane; idx < kMult * kSlice; idx += 32) {
      const int d = idx / kSlice, c = idx % kSlice;
      const long long kcol = 1ll * d * H + c0 + c;
      const float x = xs[d][c];
#pragma unroll
      for (int j = 0; j < 3; ++j) dot[j] = fmaf(x, p.fn[1ll * (warp + 8 * j) * (kMult * H) + kcol], dot[j]);
      sq = fmaf(x, x, sq);
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const float v = warp_sum(dot[j]);
      if (lane == 0) my_partial[warp + 8 * j] = v;
    }
    if (warp == 0) {
      const float v = warp_sum(sq);
      if (lane == 0) my_partial[kProj] = v;
    }
    if (warp == 1) {
      const float v = warp_sum(sqc[lane] + sqc[lane + 32] + sqc[lane + 64] + sqc[lane + 96]);
      if (lane == 0) my_partial[kProj + 1] = v;
    }
  }
  // ---------------------------------------------------------------- ticket: last block of the row finishes
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int t = atomicAdd(&p.tickets[r], 1u);
    s_last = (t == static_cast<unsigned int>(n_slices - 1)) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int j = warp; j < kStride; j += 8) {
    float acc = 0.f;
    for (int s = lane; s < n_slices; s += 32) acc += __ldcg(p.partial + (1ll * s * p.rows + r) * kStride + j);
    acc = warp_sum(acc);
    if (lane == 0) proj[j] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    const float inv = rsqrtf(proj[kProj] / (4.0f * H) + p.norm_eps);
    if (lane < 4) {
      const float a = fmaf(proj[lane] * inv, p.scale[0], p.base[lane]);
      const float b = fmaf(proj[lane + 4] * inv, p.scale[1], p.base[lane + 4]);
      p.next_pre[r * 4 + lane] = 1.0f / (1.0f + __expf(-a)) + p.hc_eps;
      p.post_out[r * 4 + lane] = 2.0f / (1.0f + __expf(-b));
    }
    float v = lane < 16 ? fmaf(proj[8 + lane] * inv, p.scale[2], p.base[8 + lane]) : 0.f;   // lane = s*4 + d
    float mx = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    v = __expf(v - mx);
    float sum = v + __shfl_xor_sync(0xffffffffu, v, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    v = v / sum + p.hc_eps;
    sum = v + __shfl_xor_sync(0xffffffffu, v, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    v /= sum + p.hc_eps;
    for (int it = 1; it < p.iters; ++it) {
      sum = v + __shfl_xor_sync(0xffffffffu, v, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      v /= sum + p.hc_eps;
      sum = v + __shfl_xor_sync(0xffffffffu, v, 4);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      v /= sum + p.hc_eps;
    }
    if (lane < 16) p.comb_out[r * 16 + lane] = v;
    if (lane == 0) p.tickets[r] = 0u;
  }
  // ---------------------------------------------------------------- RMSNorm of the collapsed row (all warps)
  const float inv = rsqrtf(proj[kProj + 1] / H + p.norm_eps);
  const int n_items = H / 8;
  for (int i = tid; i < ((n_items + 255) / 256) * 256; i += 256) {
    const bool live = i < n_items;
    float y[8];
    if (live) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(p.xc + 1ll * r * H + 8 * i));
      const float4 b = __ldcg(reinterpret_cast<const float4*>(p.xc + 1ll * r * H + 8 * i + 4));
      const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float w = p.norm_w != nullptr ? p.norm_w[8 * i + q] : 1.f;
        y[q] = bf16_round(x[q] * inv * w);
      }
      uint4 o;
      __nv_bfloat162 t0 = __floats2bfloat162_rn(y[0], y[1]), t1 = __floats2bfloat162_rn(y[2], y[3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(y[4], y[5]), t3 = __floats2bfloat162_rn(y[6], y[7]);
      o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
      o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
      *reinterpret_cast<uint4*>(p.xn + 1ll * r * H + 8 * i) = o;
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) y[q] = 0.f;
    }
    if (p.xq != nullptr) {
      // 16 consecutive lanes hold one 128-column group (H % 128 == 0 keeps groups inside `live`)
      float amax = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(y[q]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
      const float sc = fmaxf(amax * (1.0f / 448.0f), 1.17549435e-38f);
      const uint32_t bits = __float_as_uint(sc);
      uint32_t e = (bits >> 23) & 0xFF;
      if (bits & 0x7FFFFF) ++e;
      if (e > 254) e = 254;
      const float qs = __uint_as_float((254u - e) << 23);
      if (live) {
        const __nv_fp8x4_e4m3 lo(make_float4(y[0] * qs, y[1] * qs, y[2] * qs, y[3] * qs));
        const __nv_fp8x4_e4m3 hi(make_float4(y[4] * qs, y[5] * qs, y[6] * qs, y[7] * qs));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.xq + 1ll * r * H + 8 * i) = o;
        if ((i & 15) == 0) {
          uint8_t* atom = p.xq_sf + (1ll * (r / 128) * (H / 128) + i / 16) * 512;
          *reinterpret_cast<uint32_t*>(atom + (r % 32) * 16 + ((r / 32) % 4) * 4) = e * 0x01010101u;
        }
      }
    }
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_hc_step(const ds41_hc_step_args* a, void* stream) {
  if (a == nullptr || a->rows <= 0 || a->H % kSlice != 0 || a->n_ranks < 0 || a->n_ranks > 8 ||
      (a->xq != nullptr && a->xq_sf == nullptr))
    return cudaErrorInvalidValue;
  HcStepParams p{};
  p.streams_in = static_cast<const __nv_bfloat16*>(a->streams_in);
  p.streams_out = static_cast<__nv_bfloat16*>(a->streams_out);
  p.parts.n_ranks = a->n_ranks;
  p.parts.n_splits = a->n_splits;
  p.parts.split_stride = a->split_stride;
  for (int i = 0; i < a->n_ranks; ++i) p.parts.base[i] = a->part_bases[i];
  p.post = a->post; p.comb = a->comb; p.pre_in = a->pre_in;
  p.fn = a->fn; p.scale = a->scale; p.base = a->base; p.norm_w = a->norm_w;
  p.partial = a->partial; p.xc = a->xc;
  p.next_pre = a->next_pre; p.post_out = a->post_out; p.comb_out = a->comb_out;
  p.xn = static_cast<__nv_bfloat16*>(a->xn);
  p.tap_mean = a->tap_mean;
  p.xq = static_cast<uint8_t*>(a->xq);
  p.xq_sf = static_cast<uint8_t*>(a->xq_sf);
  p.tickets = a->tickets;
  p.rows = a->rows; p.H = a->H; p.iters = a->iters;
  p.hc_eps = a->hc_eps; p.norm_eps = a->norm_eps;
  p.wait_flags = a->wait_flags; p.wait_epoch = a->wait_epoch; p.status = a->status;
  return launch_pdl(hc_step_kernel, dim3(a->H / kSlice, a->rows), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant: same kernel, scratch taken from a fixed array inside the library image.
#include <atomic>

#include "ds41_noalloc.h"

namespace {
constexpr size_t kStaticPartialBytes =
    sizeof(float) * (DS41_HC_STATIC_MAX_H / ds41::kSlice) * DS41_HC_STATIC_MAX_ROWS * ds41::kStride;
constexpr size_t kStaticXcBytes = sizeof(float) * DS41_HC_STATIC_MAX_ROWS * DS41_HC_STATIC_MAX_H;
constexpr size_t kStaticTicketBytes = 256;
constexpr size_t kStaticBytes = kStaticPartialBytes + kStaticXcBytes + kStaticTicketBytes;
static_assert(kStaticPartialBytes % 256 == 0 && kStaticXcBytes % 256 == 0, "sub-buffers stay 256-byte aligned");
static_assert(sizeof(unsigned int) * DS41_HC_STATIC_MAX_ROWS <= kStaticTicketBytes, "ticket area too small");
}  // namespace

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_hc_static_scratch[kStaticBytes];

extern "C" int ds41_hc_step_static(const ds41_hc_step_args* a, void* stream) {
  if (a == nullptr || a->rows <= 0 || a->rows > DS41_HC_STATIC_MAX_ROWS || a->H <= 0 ||
      a->H > DS41_HC_STATIC_MAX_H || a->H % ds41::kSlice != 0)
    return cudaErrorInvalidValue;
  // Per-device address cache.  Threads may race to fill an entry: each looks the same symbol up with the same
  // device current and stores the same value, and the atomic makes the store and the loads well defined.  The entry
  // is never refreshed, so it goes stale if the device is reset (cudaDeviceReset) while the library stays loaded.
  static std::atomic<unsigned char*> device_base[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  unsigned char* base = device_base[dev].load(std::memory_order_acquire);
  if (base == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_hc_static_scratch);     // once per device, with that device current
    if (e != cudaSuccess) return e;
    base = static_cast<unsigned char*>(p);
    device_base[dev].store(base, std::memory_order_release);
  }
  ds41_hc_step_args b = *a;
  b.partial = reinterpret_cast<float*>(base);
  b.xc = reinterpret_cast<float*>(base + kStaticPartialBytes);
  b.tickets = reinterpret_cast<unsigned int*>(base + kStaticPartialBytes + kStaticXcBytes);
  // the array keeps whatever the previous call left: the ticket counters must start at zero
  e = cudaMemsetAsync(b.tickets, 0, kStaticTicketBytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return e;
  return ds41_hc_step(&b, stream);
}
