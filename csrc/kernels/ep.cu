// Expert-parallel token exchange over NVLink peer memory (prefill-sized MoE layers).
//
// Every rank owns e_local consecutive experts and holds `tokens` rows of the sequence.  One MoE layer is
//
//   ep_count     histogram of this rank's routes per expert; the slice for each destination rank is stored into that
//                rank's counts[src][e] (P2P stores), then phase flag 0 is raised
//   ep_plan      (as destination) waits for every source's counts, lays the received rows out as expert groups that
//                start on 128-row boundaries, stores each source's first row per expert into that source's
//                send_base[dst][e] (P2P), and writes the grouped-GEMM tile table; raises phase flag 1
//   ep_dispatch  (as source) waits for every destination's plan, then one warp per route copies the token row, its
//                route weight and its return address {source rank, token*topk+k} into the destination's receive
//                buffer (P2P 16-byte stores); the last block raises phase flag 2
//   grouped FC1 / FC2 on the tcgen05 GEMM (tile table mode): FC1 waits for phase flag 2 of all peers inside the
//                kernel; the FC2 epilogue stores every result row straight into the combine buffer of the rank the
//                token came from (P2P stores, tile by tile while other tiles still compute)
//   ep_mark      raises phase flag 3 after FC2
//   ep_combine   waits for flag 3 of all peers and sums the topk returned rows of each token in route order
//
// Row positions inside a group depend on the order in which warps take their cursor, but a row's result does not depend
// on its position and the combine sums in route order, so results are bit-reproducible.
// All waits are bounded (flag_wait_ge) and report through the status word.
// The reference has no all-to-all: its coordinator sends identical rows and routes to every expert rank over TCP/RoCE
// and sums partial planes (rust/crates/ds41rt-transport/src/v41_expert.rs:27-111, dispatch/collect/reduce wave in
// rust/crates/ds41rt-daemon/src/v41_experts/coordinator.rs; counting sort by expert in ds4_flash_aot.cu).  This file
// is the NVLink counterpart: tokens travel only to the rank that owns their expert and come back once.
#include <cuda_fp8.h>

#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

struct EpParams {
  int world, rank, e_local, topk, tokens, H, cap, bn, bn2, max_tiles, group_align;
  const __nv_bfloat16* x;
  const int* ids;
  const float* weights;
  uint32_t* epoch;
  int* cursor;
  unsigned* ticket;
  int* counts[8];
  int* send_base[8];
  __nv_bfloat16* recv_x[8];
  int2* recv_meta[8];
  float* recv_w[8];
  uint32_t* flags[8];
  int* tile_group;
  int* tile_row0;
  int* tile_end;
  int* n_tiles;
  int* total_rows;
  int* status;
  uint8_t* recv_q[8];
  uint8_t* recv_sf[8];
  int wire_fp8;
};

constexpr int kEpOverflow = 7;   // status code: received rows exceed the receive buffer

__global__ void __launch_bounds__(1024) ep_count_kernel(EpParams p) {
  extern __shared__ int hist[];
  pdl_launch_dependents();
  pdl_wait();
  const int E = p.world * p.e_local;
  for (int i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const int n = p.tokens * p.topk;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int id = p.ids[i];
    if (id >= 0 && id < E) atomicAdd(&hist[id], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const int dst = i / p.e_local;
    p.counts[dst][p.rank * p.e_local + (i - dst * p.e_local)] = hist[i];
    p.cursor[i] = 0;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    *p.ticket = 0;
    const uint32_t e = *p.epoch + 1;
    *p.epoch = e;
    __threadfence_system();
    flag_store_release(p.flags[p.rank] + 0, e);
  }
}

__global__ void __launch_bounds__(256) ep_plan_kernel(EpParams p) {
  extern __shared__ int sm[];   // [e_local] group sizes, group offsets, first tiles (two tables)
  int* gsize = sm;
  int* goff = sm + p.e_local;
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const uint32_t epoch = *p.epoch;
  if (threadIdx.x < p.world && p.world > 1) {
    if (!flag_wait_ge(p.flags[threadIdx.x] + 0, epoch, p.status, 700 + threadIdx.x)) s_ok = 0;
  }
  __syncthreads();
  const int* counts = p.counts[p.rank];
  for (int e = threadIdx.x; e < p.e_local; e += blockDim.x) {
    int g = 0;
    for (int s = 0; s < p.world; ++s) g += __ldcg(counts + s * p.e_local + e);
    gsize[e] = g;
  }
  __syncthreads();
  // table 0 (tiles of bn rows) at [0, max_tiles), table 1 (tiles of bn2 rows, if bn2 > 0) at [max_tiles, 2*max_tiles)
  int* toff = goff + p.e_local;        // [e_local] first tile of each expert, table 0
  int* toff2 = toff + p.e_local;       // same for table 1
  if (threadIdx.x == 0) {
    int off = 0, nt = 0, nt2 = 0;
    for (int e = 0; e < p.e_local; ++e) {
      goff[e] = off;
      toff[e] = nt;
      toff2[e] = nt2;
      const int g = gsize[e];
      nt += (g + p.bn - 1) / p.bn;
      if (p.bn2 > 0) nt2 += (g + p.bn2 - 1) / p.bn2;
      off += (g + p.group_align - 1) / p.group_align * p.group_align;
    }
    const bool fits = s_ok != 0 && off <= p.cap && nt <= p.max_tiles && nt2 <= p.max_tiles;
    if (!fits) {
      nt = nt2 = 0;
      if (p.status != nullptr && s_ok != 0 && atomicCAS(p.status, 0, kEpOverflow) == 0) {
        p.status[1] = 710;
        p.status[2] = off;
        p.status[3] = p.cap;
      }
      s_ok = 0;
    }
    p.n_tiles[0] = nt;
    p.n_tiles[1] = nt2;
    *p.total_rows = fits ? off : 0;
  }
  __syncthreads();
  if (s_ok) {
    for (int e = threadIdx.x; e < p.e_local; e += blockDim.x) {
      const int off = goff[e], g = gsize[e];
      int t = toff[e];
      for (int r0 = off; r0 < off + g; r0 += p.bn, ++t) {
        p.tile_group[t] = e;
        p.tile_row0[t] = r0;
        p.tile_end[t] = min(r0 + p.bn, off + g);
      }
      if (p.bn2 > 0) {
        t = p.max_tiles + toff2[e];
        for (int r0 = off; r0 < off + g; r0 += p.bn2, ++t) {
          p.tile_group[t] = e;
          p.tile_row0[t] = r0;
          p.tile_end[t] = min(r0 + p.bn2, off + g);
        }
      }
    }
  }
  __syncthreads();
  // first row of every (source, expert) run; -1 tells the source to drop the route (receive buffer too small)
  for (int i = threadIdx.x; i < p.world * p.e_local; i += blockDim.x) {
    const int src = i / p.e_local, e = i - src * p.e_local;
    int base = goff[e];
    for (int s = 0; s < src; ++s) base += __ldcg(counts + s * p.e_local + e);
    p.send_base[src][p.rank * p.e_local + e] = s_ok ? base : -1;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) flag_store_release(p.flags[p.rank] + 1, epoch);
}

__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t epoch = *p.epoch;
  if (threadIdx.x < p.world && p.world > 1) flag_wait_ge(p.flags[threadIdx.x] + 1, epoch, p.status, 720 + threadIdx.x);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int n = p.tokens * p.topk;
  const int E = p.world * p.e_local;
  const int vec = p.H / 8;   // 16-byte pieces per row
  for (int i = blockIdx.x * warps + warp; i < n; i += gridDim.x * warps) {
    const int id = p.ids[i];
    if (id < 0 || id >= E) continue;
    const int dst = id / p.e_local;
    int row = -1;
    if (lane == 0) {
      const int base = __ldcg(p.send_base[p.rank] + id);
      if (base >= 0) row = base + atomicAdd(p.cursor + id, 1);
    }
    row = __shfl_sync(0xffffffffu, row, 0);
    if (row < 0 || row >= p.cap) continue;
    const int tok = i / p.topk;
    if (p.wire_fp8) {
      // FP8 on the wire: 8 values per lane and step, one scale per 128 values (16 lanes); values and scale bytes go
      // straight into the destination's FC1 operand buffers (scale atoms of the tensor cores' block-scaled kind)
      const __nv_bfloat16* srow = p.x + 1ll * tok * p.H;
      uint8_t* qrow = p.recv_q[dst] + 1ll * row * p.H;
      uint8_t* atom_row = p.recv_sf[dst] + 1ll * (row / 128) * (p.H / 128) * 512 + (row % 32) * 16 + ((row / 32) % 4) * 4;
      for (int k0 = 0; k0 < p.H; k0 += 512) {       // two steps of 256 values in flight
        uint4 raw[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int k = k0 + u * 256 + lane * 8;
          raw[u] = k < p.H ? *reinterpret_cast<const uint4*>(srow + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int k = k0 + u * 256 + lane * 8;
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
          float f[8];
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(h[j]);
            f[2 * j] = v.x;
            f[2 * j + 1] = v.y;
            amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
          }
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
          if (k < p.H) {
            const uint32_t e = ue8m0_ceil_exp(amax * (1.0f / 448.0f));
            const float inv = __uint_as_float((254u - e) << 23);
            const __nv_fp8x4_e4m3 lo(make_float4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv));
            const __nv_fp8x4_e4m3 hi(make_float4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv));
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t*>(&lo);
            o.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(qrow + k) = o;
            if ((lane & 15) == 0) *reinterpret_cast<uint32_t*>(atom_row + 1ll * (k / 128) * 512) = e * 0x01010101u;
          }
        }
      }
      if (lane == 0) {
        p.recv_meta[dst][row] = make_int2(p.rank, i);
        p.recv_w[dst][row] = p.weights[i];
      }
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.x + 1ll * tok * p.H);
    uint4* out = reinterpret_cast<uint4*>(p.recv_x[dst] + 1ll * row * p.H);
    for (int v0 = 0; v0 < vec; v0 += 32 * 4) {      // four 16-byte loads in flight per lane
      uint4 w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int v = v0 + q * 32 + lane;
        if (v < vec) w[q] = src[v];
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int v = v0 + q * 32 + lane;
        if (v < vec) out[v] = w[q];
      }
    }
    if (lane == 0) {
      p.recv_meta[dst][row] = make_int2(p.rank, i);
      p.recv_w[dst][row] = p.weights[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(p.ticket, 1u);
    if (t == gridDim.x - 1) {
      __threadfence_system();
      flag_store_release(p.flags[p.rank] + 2, epoch);
    }
  }
}

__global__ void ep_mark_kernel(const uint32_t* epoch, uint32_t* flag) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    __threadfence_system();
    flag_store_release(flag, *epoch);
  }
}

__global__ void ep_wait_kernel(EpParams p, int phase) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x < p.world && p.world > 1)
    flag_wait_ge(p.flags[threadIdx.x] + phase, *p.epoch, p.status, 740 + 10 * phase + threadIdx.x);
}

// out[t] = sum_k comb[t*topk + k] (+ extra[t]); routes whose id is out of range contributed nothing
__global__ void __launch_bounds__(256)
ep_combine_kernel(EpParams p, const __nv_bfloat16* __restrict__ comb, const float* extra,
                  long long extra_ld, void* out, int as_bf16) {   // extra may be the output plane: coherent loads
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x < p.world && p.world > 1) flag_wait_ge(p.flags[threadIdx.x] + 3, *p.epoch, p.status, 730 + threadIdx.x);
  __syncthreads();
  const int E = p.world * p.e_local;
  const int t = blockIdx.y;
  for (int h = (blockIdx.x * blockDim.x + threadIdx.x) * 8; h < p.H; h += gridDim.x * blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = extra != nullptr ? extra[1ll * t * extra_ld + h + j] : 0.f;
    for (int k = 0; k < p.topk; ++k) {
      const int id = p.ids[t * p.topk + k];
      if (id < 0 || id >= E) continue;
      const uint4 q = __ldcg(reinterpret_cast<const uint4*>(comb + (1ll * t * p.topk + k) * p.H + h));
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (as_bf16) {
      uint4 q;
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + 1ll * t * p.H + h) = q;
    } else {
      float* o = static_cast<float*>(out) + 1ll * t * p.H + h;
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

static bool fill(const ds41_ep_args* a, EpParams& p) {
  if (a == nullptr || a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world || a->e_local < 1 ||
      a->world * a->e_local > 4096 || a->topk < 1 || a->tokens < 0 || a->H < 8 || (a->H & 7) || a->cap < 1 ||
      a->bn < 8 || a->bn2 < 0 || a->max_tiles < 1)
    return false;
  p.world = a->world; p.rank = a->rank; p.e_local = a->e_local; p.topk = a->topk; p.tokens = a->tokens;
  p.H = a->H; p.cap = a->cap; p.bn = a->bn; p.bn2 = a->bn2; p.max_tiles = a->max_tiles; p.group_align = 128;
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.ids = a->ids; p.weights = a->weights;
  p.epoch = a->epoch; p.cursor = a->cursor; p.ticket = reinterpret_cast<unsigned*>(a->ticket);
  for (int r = 0; r < 8; ++r) {
    p.counts[r] = static_cast<int*>(a->counts[r]);
    p.send_base[r] = static_cast<int*>(a->send_base[r]);
    p.recv_x[r] = static_cast<__nv_bfloat16*>(a->recv_x[r]);
    p.recv_meta[r] = static_cast<int2*>(a->recv_meta[r]);
    p.recv_w[r] = static_cast<float*>(a->recv_w[r]);
    p.flags[r] = static_cast<uint32_t*>(a->flags[r]);
  }
  p.tile_group = a->tile_group; p.tile_row0 = a->tile_row0; p.tile_end = a->tile_end;
  p.n_tiles = a->n_tiles; p.total_rows = a->total_rows; p.status = a->status;
  p.wire_fp8 = a->wire_fp8;
  for (int r = 0; r < 8; ++r) {
    p.recv_q[r] = static_cast<uint8_t*>(a->recv_q[r]);
    p.recv_sf[r] = static_cast<uint8_t*>(a->recv_sf[r]);
    if (p.wire_fp8 && r < p.world && (p.recv_q[r] == nullptr || p.recv_sf[r] == nullptr)) return false;
  }
  if (p.wire_fp8 && (p.H % 256) != 0) return false;
  return true;
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_ep_count(const ds41_ep_args* a, void* stream) {
  EpParams p;
  if (!fill(a, p)) return cudaErrorInvalidValue;
  const size_t smem = sizeof(int) * p.world * p.e_local;
  return launch_pdl(ep_count_kernel, dim3(1), dim3(1024), smem, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_ep_plan(const ds41_ep_args* a, void* stream) {
  EpParams p;
  if (!fill(a, p)) return cudaErrorInvalidValue;
  const size_t smem = sizeof(int) * 4 * p.e_local;
  return launch_pdl(ep_plan_kernel, dim3(1), dim3(256), smem, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_ep_dispatch(const ds41_ep_args* a, int blocks, void* stream) {
  EpParams p;
  if (!fill(a, p)) return cudaErrorInvalidValue;
  if (blocks < 1) blocks = 1;
  return launch_pdl(ep_dispatch_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_ep_mark(const ds41_ep_args* a, int phase, void* stream) {
  EpParams p;
  if (!fill(a, p) || phase < 0 || phase > 3) return cudaErrorInvalidValue;
  return launch_pdl(ep_mark_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint32_t*>(p.epoch), p.flags[p.rank] + phase);
}

extern "C" int ds41_ep_wait(const ds41_ep_args* a, int phase, void* stream) {
  EpParams p;
  if (!fill(a, p) || phase < 0 || phase > 3) return cudaErrorInvalidValue;
  return launch_pdl(ep_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), p, phase);
}

extern "C" int ds41_ep_combine(const ds41_ep_args* a, const void* comb, const float* extra, long long extra_ld,
                               void* out, int as_bf16, void* stream) {
  EpParams p;
  if (!fill(a, p) || comb == nullptr || out == nullptr) return cudaErrorInvalidValue;
  if (p.tokens == 0) return cudaSuccess;
  const int bx = (p.H / 8 + 255) / 256;
  return launch_pdl(ep_combine_kernel, dim3(bx, p.tokens), dim3(256), 0, static_cast<cudaStream_t>(stream), p,
                    static_cast<const __nv_bfloat16*>(comb), extra, extra_ld, out, as_bf16);
}
