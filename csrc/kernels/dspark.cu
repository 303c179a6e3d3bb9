// dSpark drafter support kernels.
//
//  taps_pack     : the target's tap means (fp32 [n_taps][rows][H]) -> bf16 rows [rows][n_taps*H] for the main projection
//  norm_rows     : sum of fp32 split planes -> RMSNorm(weight) -> bf16 rows (main_norm)
//  markov_step   : one link of the draft chain.  logits'[v] = logits[v] + <markov_head[v,:], markov_embed[prev,:]>,
//                  greedy argmax with lowest-id ties over this rank's vocabulary shard; the block that finishes
//                  last (ticket) merges the block candidates and publishes (value, token)
//                  (behaviour of the reference's draft terminal: native/cuda/kernels/v41_dspark.cu:241-290)
//  spec_feedback : prepares the next round on the device: next anchor = chosen[accepted], positions advance by
//                  accepted + 1; `forced_accept` >= 0 pins the accepted count (fixed acceptance schedule used
//                  for benchmarking with random weights)
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_philox.h"
#include "ds41_ptx.cuh"

namespace ds41 {

__global__ void taps_pack_kernel(const float* __restrict__ taps, __nv_bfloat16* __restrict__ out, int n_taps, int rows,
                                 int H, long long tap_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x;
  const long long n = 1ll * rows * n_taps * H;
  if (i >= n) return;
  const int c = static_cast<int>(i % H);
  const int t = static_cast<int>((i / H) % n_taps);
  const int r = static_cast<int>(i / (1ll * H * n_taps));
  out[i] = __float2bfloat16_rn(taps[t * tap_stride + 1ll * r * H + c]);
}

// one block (256 threads) per row; N <= 8192 and a multiple of 4.  A thread owns groups of four consecutive columns, so
// the split planes are summed with 16-byte loads (one scalar load per plane and column made the kernel a chain of 320
// dependent-latency loads per thread for 16 planes of 5120 columns).
__global__ void __launch_bounds__(256) norm_rows_kernel(const float* __restrict__ planes, int splits, long long plane,
                                                        const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                        int N, float eps) {
  __shared__ float part[8];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  float4 vals[8];
  float sq = 0.f;
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int c = 4 * (tid + 256 * n);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < N) {
#pragma unroll 4
      for (int s = 0; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(planes + s * plane + 1ll * r * N + c);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      a = make_float4(bf16_round(a.x), bf16_round(a.y), bf16_round(a.z), bf16_round(a.w));
    }
    vals[n] = a;
    sq = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, sq))));
  }
  sq = warp_sum(sq);
  if ((tid & 31) == 0) part[tid >> 5] = sq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += part[i];
  const float inv = rsqrtf(tot / N + eps);
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int c = 4 * (tid + 256 * n);
    if (c < N) {
      const float4 g = w != nullptr ? *reinterpret_cast<const float4*>(w + c) : make_float4(1.f, 1.f, 1.f, 1.f);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(vals[n].x * inv * g.x, vals[n].y * inv * g.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(vals[n].z * inv * g.z, vals[n].w * inv * g.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(out + 1ll * r * N + c) = o;
    }
  }
}

struct MarkovParams {
  const float* logits;            // [V_local] base logits of this draft row
  const __nv_bfloat16* head;      // [V_local][rank]
  const __nv_bfloat16* embed;     // [V][rank]
  const int* prev_token;          // device scalar: token that precedes this draft position
  int v_local, v_offset, rank, vocab;
  float* block_val;               // [gridDim.x]
  int* block_idx;
  unsigned int* ticket;           // zero before first use; reset by the finishing block
  float* best_val;                // [1]
  int* best_idx;                  // [1] global token id
  // draft sampling: temperature > 0 turns the arg max into a Gumbel-max draw, key = x / T - log(-log(u)), with
  // u = Philox(seed, subsequence, offset + token / 4)[token % 4]; temperature <= 0 is greedy
  float temperature;
  unsigned long long seed, subsequence, offset;
};

// grid: enough blocks of 256 threads; each warp strides over vocabulary rows. rank <= 256, multiple of 8.
// kSample = false is the greedy form: without the counter-based generator in the loop the kernel needs half the
// registers, and twice the warps per SM hide the row loads' latency.
template <bool kSample>
__global__ void __launch_bounds__(256, 3) markov_step_kernel(MarkovParams p) {
  __shared__ float e[256];
  __shared__ float wv[8];
  __shared__ int wi[8];
  __shared__ int s_last;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int prev = *p.prev_token;
  if (prev < 0 || prev >= p.vocab) prev = 0;
  if (tid < p.rank) e[tid] = __bfloat162float(p.embed[1ll * prev * p.rank + tid]);
  __syncthreads();
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int lanes_per_row = p.rank / 8;             // 8 bf16 (16 B) per lane
  const int rows_per_warp = 32 / lanes_per_row;     // rank 256 -> 1 row per warp pass; rank 64 -> 4
  const int sub = lane / lanes_per_row, l = lane % lanes_per_row;
  // Every warp owns a contiguous run of row groups and walks it eight groups at a time: the eight 16-byte loads of a
  // lane (and the base logits of those rows) are issued before the first dot product.  With one row in flight per warp
  // the kernel waited out a memory latency per row and ran at a fifth of the copy bandwidth.
  constexpr int kBatch = 8;
  const int groups = (p.v_local + rows_per_warp - 1) / rows_per_warp;
  const int n_warps = gridDim.x * 8;
  const int per_warp = (groups + n_warps - 1) / n_warps;
  const int g_begin = (blockIdx.x * 8 + warp) * per_warp, g_end = min(groups, g_begin + per_warp);
  for (int g0 = g_begin; g0 < g_end; g0 += kBatch) {
    uint4 raw[kBatch];
    float base[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = (g0 + u) * rows_per_warp + sub;
      const bool live = g0 + u < g_end && v < p.v_local && sub < rows_per_warp;
      raw[u] = live ? *reinterpret_cast<const uint4*>(p.head + 1ll * v * p.rank + l * 8) : make_uint4(0u, 0u, 0u, 0u);
      base[u] = (live && l == 0) ? p.logits[v] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
      float acc = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc = fmaf(f.x, e[l * 8 + 2 * q], fmaf(f.y, e[l * 8 + 2 * q + 1], acc));
      }
      for (int o = lanes_per_row / 2; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const int v = (g0 + u) * rows_per_warp + sub;
      if (l == 0 && g0 + u < g_end && v < p.v_local && sub < rows_per_warp) {
        float x = base[u] + acc;
        const int tok = p.v_offset + v;
        if constexpr (kSample) {
          const Philox4 rnd = philox4x32_10(p.seed, p.subsequence, p.offset + static_cast<unsigned long long>(tok >> 2));
          const float u01 = philox_uniform(rnd.v[tok & 3]);
          x = x / p.temperature - __logf(-__logf(u01));
        }
        if (x > best || (x == best && tok < best_i)) { best = x; best_i = tok; }
      }
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w)
      if (wv[w] > best || (wv[w] == best && wi[w] < best_i)) { best = wv[w]; best_i = wi[w]; }
    p.block_val[blockIdx.x] = best;
    p.block_idx[blockIdx.x] = best_i;
    __threadfence();
    const unsigned int t = atomicAdd(p.ticket, 1u);
    s_last = (t == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  best = -INFINITY;
  best_i = 0x7fffffff;
  for (int b = tid; b < static_cast<int>(gridDim.x); b += 256) {
    const float ov = __ldcg(p.block_val + b);
    const int oi = __ldcg(p.block_idx + b);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w)
      if (wv[w] > best || (wv[w] == best && wi[w] < best_i)) { best = wv[w]; best_i = wi[w]; }
    *p.best_val = best;
    *p.best_idx = best_i == 0x7fffffff ? -1 : best_i;
    *p.ticket = 0u;
  }
}

struct SpecFeedbackParams {
  const int* inputs;      // [width] tokens the verification pass consumed (anchor, drafts...)
  const int* chosen;      // [width] target's choice after each row
  int width, forced_accept, eos;
  int* accepted;          // [1]
  int* emitted;           // [width] tokens emitted this round (chosen[0..accepted])
  int* n_emitted;         // [1]
  int* next_anchor;       // [1]
  int* target_pos;        // [>= width]: verification rows' positions, advanced for the next round
  int* draft_pos;         // [>= width]: drafter rows' positions
  int* draft_hi;          // [>= width]: drafter rows' highest visible position
  int* target_tokens;     // [>= width]: row 0 receives the next anchor
  int* draft_tokens;      // [>= width]: row 0 receives the next anchor
  long long* total_emitted;   // running counter
};
__global__ void spec_feedback_kernel(SpecFeedbackParams p) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int acc = 0;
  if (p.forced_accept >= 0) {
    acc = min(p.forced_accept, p.width - 1);
  } else {
    while (acc + 1 < p.width && p.inputs[acc + 1] == p.chosen[acc] && p.chosen[acc] != p.eos) ++acc;
  }
  for (int j = 0; j <= acc; ++j) p.emitted[j] = p.chosen[j];
  *p.accepted = acc;
  *p.n_emitted = acc + 1;
  const int anchor = p.chosen[acc];
  *p.next_anchor = anchor;
  p.target_tokens[0] = anchor;
  p.draft_tokens[0] = anchor;
  const int base = p.target_pos[0] + acc + 1;
  for (int j = 0; j < p.width; ++j) {
    p.target_pos[j] = base + j;
    p.draft_pos[j] = base + j;
    p.draft_hi[j] = base + p.width - 1;
  }
  if (p.total_emitted != nullptr) *p.total_emitted += acc + 1;
}

// copy `n` ints device-to-device with an element offset (draft tokens -> verification inputs)
__global__ void copy_ints_kernel(const int* src, int* dst, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i];
}

// ---- confidence head: raw projection of [collapsed hidden row | Markov embedding of the previous token] per draft row.
// Row j's previous token is the anchor (j = 0) or draft j - 1.  The consumer applies the sigmoid.
// Reference: native/cuda/kernels/v41_dspark.cu:40-58 (same inputs, promoted to fp32, one block per row).
__global__ void __launch_bounds__(256) confidence_kernel(const float* __restrict__ hidden, long long ld_hidden,
                                                         const __nv_bfloat16* __restrict__ embed, int rank,
                                                         const int* __restrict__ anchor, const int* __restrict__ drafts,
                                                         const __nv_bfloat16* __restrict__ weight, float* __restrict__ out,
                                                         int H, int vocab) {
  __shared__ float partial[8];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  int prev = row == 0 ? anchor[0] : drafts[row - 1];
  prev = min(max(prev, 0), vocab - 1);
  float sum = 0.f;
  for (int c = tid; c < H + rank; c += 256) {
    const float x = c < H ? hidden[row * ld_hidden + c] : __bfloat162float(embed[1ll * prev * rank + (c - H)]);
    sum = fmaf(x, __bfloat162float(weight[c]), sum);
  }
  sum = warp_sum(sum);
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    sum = warp_sum(lane < 8 ? partial[lane] : 0.f);
    if (lane == 0) out[row] = sum;
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_dspark_confidence(const float* hidden, long long ld_hidden, const void* embed, int rank,
                                      const int* anchor, const int* drafts, const void* weight, float* out, int rows,
                                      int H, int vocab, void* stream) {
  if (rows <= 0 || H <= 0 || rank <= 0 || vocab <= 0) return cudaErrorInvalidValue;
  return launch_pdl(confidence_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), hidden, ld_hidden,
                    static_cast<const __nv_bfloat16*>(embed), rank, anchor, drafts,
                    static_cast<const __nv_bfloat16*>(weight), out, H, vocab);
}

extern "C" int ds41_taps_pack(const float* taps, void* out, int n_taps, int rows, int H, long long tap_stride,
                              void* stream) {
  if (n_taps <= 0 || rows <= 0 || H <= 0) return cudaErrorInvalidValue;
  const long long n = 1ll * rows * n_taps * H;
  return launch_pdl(taps_pack_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), taps, static_cast<__nv_bfloat16*>(out), n_taps, rows, H,
                    tap_stride);
}

extern "C" int ds41_norm_rows(const float* planes, int splits, long long plane, const float* w, void* out, int rows,
                              int N, float eps, void* stream) {
  if (rows <= 0 || N <= 0 || N > 8192 || (N & 3) || (plane & 3) || splits <= 0) return cudaErrorInvalidValue;
  return launch_pdl(norm_rows_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), planes, splits,
                    plane, w, static_cast<__nv_bfloat16*>(out), N, eps);
}

extern "C" int ds41_markov_step(const float* logits, const void* head, const void* embed, const int* prev_token,
                                int v_local, int v_offset, int rank, int vocab, float* block_val, int* block_idx,
                                int n_blocks, unsigned int* ticket, float* best_val, int* best_idx,
                                const ds41_draft_rng* rng, void* stream) {
  if (v_local <= 0 || rank <= 0 || rank > 256 || (rank & 7) || (32 % (rank / 8)) != 0 || n_blocks <= 0)
    return cudaErrorInvalidValue;
  MarkovParams p{logits, static_cast<const __nv_bfloat16*>(head), static_cast<const __nv_bfloat16*>(embed),
                 prev_token, v_local, v_offset, rank, vocab, block_val, block_idx, ticket, best_val, best_idx,
                 rng != nullptr ? rng->temperature : 0.f, rng != nullptr ? rng->seed : 0ull,
                 rng != nullptr ? rng->subsequence : 0ull, rng != nullptr ? rng->offset : 0ull};
  if (p.temperature > 0.f)
    return launch_pdl(markov_step_kernel<true>, dim3(n_blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
  return launch_pdl(markov_step_kernel<false>, dim3(n_blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_spec_feedback(const int* inputs, const int* chosen, int width, int forced_accept, int eos,
                                  int* accepted, int* emitted, int* n_emitted, int* next_anchor, int* target_pos,
                                  int* draft_pos, int* draft_hi, int* target_tokens, int* draft_tokens,
                                  long long* total_emitted, void* stream) {
  if (width <= 0) return cudaErrorInvalidValue;
  SpecFeedbackParams p{inputs, chosen, width, forced_accept, eos, accepted, emitted, n_emitted, next_anchor,
                       target_pos, draft_pos, draft_hi, target_tokens, draft_tokens, total_emitted};
  return launch_pdl(spec_feedback_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_copy_ints(const int* src, int* dst, int n, void* stream) {
  if (n <= 0) return cudaErrorInvalidValue;
  return launch_pdl(copy_ints_kernel, dim3((n + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), src, dst,
                    n);
}
