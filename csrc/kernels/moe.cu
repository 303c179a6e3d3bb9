// Router, decode-side expert planning and combine.
//
//  router_select : reduce split-K planes of [gate logits | shared gate | shared up], score = sqrt(softplus),
//                  biased top-k (lowest id wins ties), weights = score / (sum + 1e-20) * route_scale, and the
//                  shared expert's clamp-SwiGLU activation (native/cuda/kernels/v41_router.cu:13-112,
//                  v41_fp8.cu:14-21)
//  moe_plan      : from the (row, k) routes build this rank's ascending list of active local experts and a
//                  dense [active][row] weight table (0 = row not routed to that expert).  The grouped FC1/FC2
//                  GEMMs run every active expert against all rows of the small decode batch and mask with
//                  this table, so no token gather is needed on the decode path.
//  moe_combine   : per row, fixed-order sum of its routes' FC2 rows plus the shared expert's split planes ->
//                  this rank's fp32 partial plane (the cross-rank sum happens in hc_post_mix).
//                  (reduction-order contract of native/cuda/kernels/v41_route_reduce.cu:13-34)
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

struct RouterParams {
  const float* planes;    // [splits][rows][ntot]: columns [0,E) gate logits, then I_sh gate, I_sh up
  int splits, rows, ntot, E, I_sh, topk;
  const float* bias;      // [E]
  float route_scale, limit;
  int* ids;               // [rows][topk]
  float* weights;         // [rows][topk]
  __nv_bfloat16* shared_act;   // [rows][I_sh]
};

// one block of 512 threads per row; E <= 512
__global__ void __launch_bounds__(512) router_select_kernel(RouterParams p) {
  __shared__ float score[512];
  __shared__ float biased[512];
  __shared__ float wmax[16];
  __shared__ int widx[16];
  __shared__ int chosen[16];
  __shared__ float chosen_score[16];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const long long plane = 1ll * p.rows * p.ntot;
  const float* row0 = p.planes + 1ll * r * p.ntot;
  if (blockIdx.y == 1) {
    // second block of the row: the shared expert's clamp-SwiGLU activation
    for (int i = tid; i < p.I_sh; i += 512) {
      float g = 0.f, u = 0.f;
#pragma unroll 4
      for (int s = 0; s < p.splits; ++s) {
        g += row0[s * plane + p.E + i];
        u += row0[s * plane + p.E + p.I_sh + i];
      }
      g = fminf(bf16_round(g), p.limit);
      u = fminf(fmaxf(bf16_round(u), -p.limit), p.limit);
      p.shared_act[1ll * r * p.I_sh + i] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
    }
    return;
  }
  if (tid < p.E) {
    float a = 0.f;
#pragma unroll 4
    for (int s = 0; s < p.splits; ++s) a += row0[s * plane + tid];
    const float sp = a > 20.f ? a : log1pf(__expf(a));
    const float sc = sqrtf(sp);
    score[tid] = sc;
    biased[tid] = sc + p.bias[tid];
  } else {
    score[tid] = 0.f;
    biased[tid] = -INFINITY;
  }
  __syncthreads();
  for (int k = 0; k < p.topk; ++k) {
    float v = biased[tid];
    int i = tid;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    if (lane == 0) { wmax[warp] = v; widx[warp] = i; }
    __syncthreads();
    if (tid == 0) {
      float bv = wmax[0];
      int bi = widx[0];
      for (int w = 1; w < 16; ++w)
        if (wmax[w] > bv || (wmax[w] == bv && widx[w] < bi)) { bv = wmax[w]; bi = widx[w]; }
      chosen[k] = bi;
      chosen_score[k] = score[bi];
      biased[bi] = -INFINITY;
    }
    __syncthreads();
  }
  if (tid == 0) {
    float sum = 0.f;
    for (int k = 0; k < p.topk; ++k) sum += chosen_score[k];
    for (int k = 0; k < p.topk; ++k) {
      p.ids[r * p.topk + k] = chosen[k];
      p.weights[r * p.topk + k] = chosen_score[k] / (sum + 1e-20f) * p.route_scale;
    }
  }
}

struct PlanParams {
  const int* ids;         // [rows][topk]
  const float* weights;
  const int* row_slot;    // rows with slot < 0 are padding and route nowhere
  int rows, topk, e0, e1; // this rank owns experts [e0, e1)
  int max_active, row_w_ld;
  int* active;            // [max_active] local expert index (ascending)
  int* n_active;          // [1]
  float* row_w;           // [max_active][row_w_ld]
  int* slot_of;           // [rows][topk] index into `active`, -1 if not local
};

// single block, 512 threads; (e1 - e0) <= 512
__global__ void __launch_bounds__(512) moe_plan_kernel(PlanParams p) {
  __shared__ int used[512];
  __shared__ int slot_of_expert[512];
  __shared__ int warp_tot[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  used[tid] = 0;
  __syncthreads();
  for (int i = tid; i < p.rows * p.topk; i += 512) {
    const int e = p.ids[i];
    if (p.row_slot[i / p.topk] >= 0 && e >= p.e0 && e < p.e1) used[e - p.e0] = 1;
  }
  __syncthreads();
  // exclusive scan of `used` -> slot numbers in ascending expert order
  const int v = used[tid];
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int w = 0; w < 16; ++w) { const int t = warp_tot[w]; warp_tot[w] = run; run += t; }
    *p.n_active = min(run, p.max_active);
  }
  __syncthreads();
  const int slot = warp_tot[warp] + incl - v;
  slot_of_expert[tid] = (v && slot < p.max_active) ? slot : -1;
  if (v && slot < p.max_active) p.active[slot] = tid;
  __syncthreads();
  for (int i = tid; i < p.max_active * p.row_w_ld; i += 512) p.row_w[i] = 0.f;
  __syncthreads();
  for (int i = tid; i < p.rows * p.topk; i += 512) {
    const int e = p.ids[i];
    int s = -1;
    if (p.row_slot[i / p.topk] >= 0 && e >= p.e0 && e < p.e1) s = slot_of_expert[e - p.e0];
    p.slot_of[i] = s;
    if (s >= 0) p.row_w[1ll * s * p.row_w_ld + i / p.topk] = p.weights[i];
  }
}

struct CombineParams {
  const float* fc2;         // [max_active][rows][H]
  const int* slot_of;       // [rows][topk]
  const float* shared;      // [shared_splits][rows][H] or null
  int shared_splits;
  int rows, topk, H;
  float* out;               // [rows][H]
  unsigned int* counter;    // optional: completion signal (see publish_all)
  uint32_t* epoch;
  uint32_t* const* flags;
  int n_flags;
};

// The block that arrives last publishes "this rank's planes are complete": it bumps the rank's epoch and stores the
// new value into its slot of every rank's flag array (so that every rank polls its own memory).  Call it after the
// block's stores, from every thread.
__device__ __forceinline__ void publish_all(unsigned int* counter, uint32_t* epoch, uint32_t* const* flags,
                                            int n_flags, unsigned int n_blocks) {
  __shared__ unsigned int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(counter, 1u) == n_blocks - 1 ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 32) {
    uint32_t e = 0;
    if (threadIdx.x == 0) {
      e = *epoch + 1;
      *epoch = e;
      *counter = 0u;
    }
    e = __shfl_sync(0xffffffffu, e, 0);
    // one release store per flag: it orders this rank's earlier plane writes (observed through the counter and the
    // fence above) before the flag at system scope; no separate system fence is needed in front of it
    if (static_cast<int>(threadIdx.x) < n_flags) flag_store_release(flags[threadIdx.x], e);
  }
}

__global__ void __launch_bounds__(256) moe_combine_kernel(CombineParams p) {
  const int r = blockIdx.y;
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  pdl_launch_dependents();
  pdl_wait();
  if (c < p.H) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < p.topk; ++k) {
      const int s = p.slot_of[r * p.topk + k];
      if (s >= 0) {
        const float4 v = *reinterpret_cast<const float4*>(p.fc2 + (1ll * s * p.rows + r) * p.H + c);
        // per-route bf16 boundary, then fp32 accumulation in route order
        acc.x += bf16_round(v.x); acc.y += bf16_round(v.y); acc.z += bf16_round(v.z); acc.w += bf16_round(v.w);
      }
    }
    for (int s = 0; s < p.shared_splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(p.shared + (1ll * s * p.rows + r) * p.H + c);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(p.out + 1ll * r * p.H + c) = acc;
  }
  if (p.counter != nullptr) publish_all(p.counter, p.epoch, p.flags, p.n_flags, gridDim.x * gridDim.y);
}

// ---- the same publication as a kernel of its own (after kernels that do not fold it in)
__global__ void signal_all_kernel(unsigned int* epoch, uint32_t* const* flags, int n) {
  pdl_launch_dependents();
  pdl_wait();
  uint32_t e = 0;
  if (threadIdx.x == 0) {
    e = *epoch + 1;
    *epoch = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  if (static_cast<int>(threadIdx.x) < n) flag_store_release(flags[threadIdx.x], e);
}

// ---- publish "this rank's partial planes are complete": bump the rank-local epoch and store it to the flag
__global__ void signal_kernel(uint32_t* epoch, uint32_t* flag) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    const uint32_t e = *epoch + 1;
    *epoch = e;
    __threadfence_system();
    flag_store_release(flag, e);
  }
}

// ---- reduce fp32 split planes into one bf16 (or fp32) matrix
__global__ void reduce_planes_kernel(const float* planes, int splits, long long plane, void* out, int as_bf16,
                                     long long n) {
  const long long i = (1ll * blockIdx.x * blockDim.x + threadIdx.x) * 2;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= n) return;
  float a = 0.f, b = 0.f;
  for (int s = 0; s < splits; ++s) {
    a += planes[s * plane + i];
    if (i + 1 < n) b += planes[s * plane + i + 1];
  }
  if (as_bf16) {
    if (i + 1 < n) reinterpret_cast<__nv_bfloat162*>(out)[i / 2] = __floats2bfloat162_rn(a, b);
    else static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(a);
  } else {
    static_cast<float*>(out)[i] = a;
    if (i + 1 < n) static_cast<float*>(out)[i + 1] = b;
  }
}

// ---- split-K planes of a grouped projection, [split][group][rows][width] fp32 -> bf16 [rows][ld_out] with group g in
// columns [g * width, (g + 1) * width); the splits are summed in order
__global__ void reduce_groups_kernel(const float* planes, int splits, int groups, int rows, int width,
                                     __nv_bfloat16* out, long long ld_out) {
  const long long i = (1ll * blockIdx.x * blockDim.x + threadIdx.x) * 2;
  pdl_launch_dependents();
  pdl_wait();
  const long long per_split = 1ll * groups * rows * width;
  if (i >= per_split) return;
  float a = 0.f, b = 0.f;
#pragma unroll 4
  for (int s = 0; s < splits; ++s) {
    const float2 v = *reinterpret_cast<const float2*>(planes + s * per_split + i);
    a += v.x;
    b += v.y;
  }
  const int c = static_cast<int>(i % width);
  const long long gr = i / width;
  const int r = static_cast<int>(gr % rows), g = static_cast<int>(gr / rows);
  *reinterpret_cast<__nv_bfloat162*>(out + r * ld_out + 1ll * g * width + c) = __floats2bfloat162_rn(a, b);
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_reduce_groups(const float* planes, int splits, int groups, int rows, int width, void* out,
                                  long long ld_out, void* stream) {
  if (splits <= 0 || groups <= 0 || rows <= 0 || width <= 0 || (width & 1) || (ld_out & 1)) return cudaErrorInvalidValue;
  const long long threads = 1ll * groups * rows * width / 2;
  return launch_pdl(reduce_groups_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), planes, splits, groups, rows, width,
                    static_cast<__nv_bfloat16*>(out), ld_out);
}

extern "C" int ds41_router_select(const float* planes, int splits, int rows, int ntot, int E, int I_sh, int topk,
                                  const float* bias, float route_scale, float limit, int* ids, float* weights,
                                  void* shared_act, void* stream) {
  if (rows <= 0 || E > 512 || topk > 16 || E + 2 * I_sh > ntot) return cudaErrorInvalidValue;
  RouterParams p{planes, splits, rows, ntot, E, I_sh, topk, bias, route_scale, limit, ids, weights,
                 static_cast<__nv_bfloat16*>(shared_act)};
  return launch_pdl(router_select_kernel, dim3(rows, I_sh > 0 ? 2 : 1), dim3(512), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_moe_plan(const int* ids, const float* weights, const int* row_slot, int rows, int topk, int e0,
                             int e1, int max_active, int row_w_ld, int* active, int* n_active, float* row_w,
                             int* slot_of, void* stream) {
  if (rows <= 0 || e1 - e0 > 512 || e1 <= e0 || row_w_ld < rows) return cudaErrorInvalidValue;
  PlanParams p{ids, weights, row_slot, rows, topk, e0, e1, max_active, row_w_ld, active, n_active, row_w, slot_of};
  return launch_pdl(moe_plan_kernel, dim3(1), dim3(512), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_moe_combine(const float* fc2, const int* slot_of, const float* shared, int shared_splits,
                                int rows, int topk, int H, float* out, void* stream) {
  if (rows <= 0 || (H & 3)) return cudaErrorInvalidValue;
  CombineParams p{fc2, slot_of, shared, shared_splits, rows, topk, H, out, nullptr, nullptr, nullptr, 0};
  dim3 grid((H / 4 + 255) / 256, rows);
  return launch_pdl(moe_combine_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_moe_combine_signal(const float* fc2, const int* slot_of, const float* shared, int shared_splits,
                                       int rows, int topk, int H, float* out, unsigned int* counter, uint32_t* epoch,
                                       uint32_t* const* flags, int n_flags, void* stream) {
  if (rows <= 0 || (H & 3) || counter == nullptr || epoch == nullptr || flags == nullptr || n_flags <= 0 || n_flags > 32)
    return cudaErrorInvalidValue;
  CombineParams p{fc2, slot_of, shared, shared_splits, rows, topk, H, out, counter, epoch, flags, n_flags};
  dim3 grid((H / 4 + 255) / 256, rows);
  return launch_pdl(moe_combine_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_signal_all(uint32_t* epoch, uint32_t* const* flags, int n, void* stream) {
  if (epoch == nullptr || flags == nullptr || n <= 0 || n > 32) return cudaErrorInvalidValue;
  return launch_pdl(signal_all_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), epoch, flags, n);
}

extern "C" int ds41_signal(uint32_t* epoch, uint32_t* flag, void* stream) {
  return launch_pdl(signal_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), epoch, flag);
}

extern "C" int ds41_reduce_planes(const float* planes, int splits, long long plane, void* out, int as_bf16,
                                  long long n, void* stream) {
  if (n <= 0 || splits <= 0) return cudaErrorInvalidValue;
  const long long threads = (n + 1) / 2;
  return launch_pdl(reduce_planes_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), planes, splits, plane, out, as_bf16, n);
}
