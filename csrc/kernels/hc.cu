// Hyper-connection (mHC) kernels and the embedding fan-out.
//
// Residual state is `mult` (=4) streams per token: streams[rows][mult][H] bf16.  Per sublayer:
//   mixes    : proj = (flat(streams) . fn[j]) * rsqrt(mean(flat^2)+norm_eps), j < 2*mult + mult^2
//              pre  = sigmoid(proj*scale0+base)+eps, post = 2*sigmoid(proj*scale1+base),
//              comb = Sinkhorn(softmax rows), indexed [source][destination]
//   collapse : x = sum_s pre_in[s]*streams[s]  (pre_in comes from the PREVIOUS sublayer's mixes)
//   expand   : streams'[d] = post[d]*sublayer + sum_s comb[s][d]*streams[s]
// (behaviour of the reference's native/cuda/kernels/v41_hc.cu:6-29,70-120 and
//  rust/crates/ds41rt-daemon/src/v41_hc.rs:153-225).
//
// Layout of the fused pipeline here:
//   hc_post_mix  : expand with the sublayer output given as a sum of partial planes (this GPU's split-K
//                  planes and, for tensor parallelism, every peer's planes read over NVLink), write the new
//                  streams, and accumulate this column slice's contribution to the NEXT mixes projection.
//   hc_finish    : reduce the slice partials in fixed order, compute pre/post/comb, collapse with the
//                  incoming pre and apply the RMSNorm weight -> normalised bf16 rows for the GEMMs.
// Long passes put the mixes projection on the tensor cores instead: hc_post_mix runs without `fn` (expand, store and
// the row's sum of squares only), a tcgen05 GEMM multiplies the stored streams [rows, 4H] by the mixing matrix given as
// bf16 high and low parts ([24 high | 24 low | pad] x 4H, so the sum carries about 16 mantissa bits of the fp32
// matrix), and hc_finish adds the two parts of every split-K plane.  24 dot products of length 4H per row are
// 4 GFMA for 8192 rows: as SIMT work they made this the second largest kernel of a prompt pass.
#include <atomic>

#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

constexpr int kHcMaxMult = 4;
constexpr int kHcProj = 2 * kHcMaxMult + kHcMaxMult * kHcMaxMult;   // 24
constexpr int kHcSlice = 128;                                       // columns of H per block
constexpr int kHcRowsPerBlock = 8;                                  // 8 rows x 32 four-column groups = one item per thread
constexpr int kHcPartialStride = kHcProj + 1;                       // 24 dots + sum of squares

struct PartList {
  const float* base[8];     // per rank: planes [n_splits][rows][H] fp32
  int n_ranks;
  int n_splits;
  long long split_stride;   // elements between split planes
};

__global__ void embed_streams_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ embed,
                                     __nv_bfloat16* __restrict__ streams, float* __restrict__ pre, int rows, int H,
                                     int mult, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  int tok = tokens[r];
  if (tok < 0 || tok >= vocab) tok = 0;
  const uint4* src = reinterpret_cast<const uint4*>(embed + 1ll * tok * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = src[i];
    for (int s = 0; s < mult; ++s) reinterpret_cast<uint4*>(streams + (1ll * r * mult + s) * H)[i] = v;
  }
  if (threadIdx.x < mult) pre[r * mult + threadIdx.x] = threadIdx.x == 0 ? 1.0f : 0.0f;
}

// grid (H / kHcSlice, ceil(rows / kHcRowsPerBlock)), 256 threads.
// parts.n_ranks == 0: no expand, mixes are computed on `streams_in` as they are.
__global__ void __launch_bounds__(256)
hc_post_mix_kernel(const __nv_bfloat16* streams_in, __nv_bfloat16* streams_out,   // same buffer in the engine: coherent loads
                   PartList parts, const float* __restrict__ post, const float* __restrict__ comb,
                   const float* __restrict__ fn, float* __restrict__ partial, int rows, int H,
                   const uint32_t* const* __restrict__ wait_flags, const uint32_t* __restrict__ wait_epoch, int* status,
                   int rows_per_block) {
  // The block's slice of the mixing matrix (24 projections x 4 streams x 128 columns, 48 KB) stays in shared memory
  // while the block walks `rows_per_block` rows in groups of eight: fetched per group it was four times the stream
  // bytes the group itself moves, and the kernel ran at a sixth of the copy bandwidth.
  extern __shared__ __align__(16) float hc_smem[];
  float (*xs)[kHcMaxMult][kHcSlice] = reinterpret_cast<float (*)[kHcMaxMult][kHcSlice]>(hc_smem);
  float* fs = hc_smem + kHcRowsPerBlock * kHcMaxMult * kHcSlice;      // [24][4 * 128]
  const int c0 = blockIdx.x * kHcSlice;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < kHcProj * kHcMaxMult * (kHcSlice / 4); i += blockDim.x) {     // weights: before the dependency wait
    const int j = i / (kHcMaxMult * (kHcSlice / 4)), rem = i % (kHcMaxMult * (kHcSlice / 4));
    const int d = rem / (kHcSlice / 4), c4 = (rem % (kHcSlice / 4)) * 4;
    *reinterpret_cast<float4*>(fs + j * (kHcMaxMult * kHcSlice) + d * kHcSlice + c4) =
        *reinterpret_cast<const float4*>(fn + 1ll * j * (kHcMaxMult * H) + 1ll * d * H + c0 + c4);
  }
  pdl_launch_dependents();
  pdl_wait();

  if (wait_flags != nullptr && parts.n_ranks > 1) {
    // every peer publishes "my partial planes for this step are complete" by raising its flag
    if (tid < parts.n_ranks) flag_wait_ge(wait_flags[tid], *wait_epoch, status, 400 + tid);
    __syncthreads();
  }
  const int r_begin = blockIdx.y * rows_per_block, r_end = min(rows, r_begin + rows_per_block);
  for (int r0 = r_begin; r0 < r_end; r0 += kHcRowsPerBlock) {
  if (r0 > r_begin) __syncthreads();                  // the previous group's rows have been read by every warp
  // ---- expand (or plain load) into shared memory, bf16-rounded like the stored streams.  One item = one row x four
  // adjacent columns: 8-byte stream loads and 16-byte plane loads, all issued before the first use.
  for (int idx = tid; idx < kHcRowsPerBlock * (kHcSlice / 4); idx += blockDim.x) {
    const int rr = idx / (kHcSlice / 4), c = (idx % (kHcSlice / 4)) * 4;
    const int r = r0 + rr;
    float out[kHcMaxMult][4];
#pragma unroll
    for (int d = 0; d < kHcMaxMult; ++d)
#pragma unroll
      for (int j = 0; j < 4; ++j) out[d][j] = 0.f;
    if (r < rows) {
      float s_in[kHcMaxMult][4];
#pragma unroll
      for (int s = 0; s < kHcMaxMult; ++s) {
        const uint2 raw = *reinterpret_cast<const uint2*>(streams_in + (1ll * r * kHcMaxMult + s) * H + c0 + c);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        s_in[s][0] = lo.x; s_in[s][1] = lo.y; s_in[s][2] = hi.x; s_in[s][3] = hi.y;
      }
      if (parts.n_ranks > 0) {
        float sub[4] = {0.f, 0.f, 0.f, 0.f};
        // rank-major, split-minor order; eight plane loads in flight before the first add (peer loads are slow)
        const int n_sp = parts.n_splits, total = parts.n_ranks * n_sp;
        for (int j0 = 0; j0 < total; j0 += 8) {
          float4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int j = j0 + u;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j < total) {
              const int k = j / n_sp, sp = j - k * n_sp;
              v[u] = __ldcg(reinterpret_cast<const float4*>(parts.base[k] + sp * parts.split_stride +
                                                            1ll * r * H + c0 + c));
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) { sub[0] += v[u].x; sub[1] += v[u].y; sub[2] += v[u].z; sub[3] += v[u].w; }
        }
        float cm[16], pw[4];
#pragma unroll
        for (int q = 0; q < 16; ++q) cm[q] = comb[r * 16 + q];
#pragma unroll
        for (int q = 0; q < 4; ++q) pw[q] = post[r * 4 + q];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float sb = bf16_round(sub[j]);
#pragma unroll
          for (int d = 0; d < kHcMaxMult; ++d) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < kHcMaxMult; ++s) acc = fmaf(cm[s * 4 + d], s_in[s][j], acc);
            out[d][j] = bf16_round(fmaf(pw[d], sb, acc));
          }
        }
#pragma unroll
        for (int d = 0; d < kHcMaxMult; ++d) {
          const __nv_bfloat162 a = __floats2bfloat162_rn(out[d][0], out[d][1]);
          const __nv_bfloat162 b = __floats2bfloat162_rn(out[d][2], out[d][3]);
          uint2 w;
          w.x = *reinterpret_cast<const uint32_t*>(&a);
          w.y = *reinterpret_cast<const uint32_t*>(&b);
          *reinterpret_cast<uint2*>(streams_out + (1ll * r * kHcMaxMult + d) * H + c0 + c) = w;
        }
      } else {
#pragma unroll
        for (int d = 0; d < kHcMaxMult; ++d)
#pragma unroll
          for (int j = 0; j < 4; ++j) out[d][j] = s_in[d][j];
      }
    }
#pragma unroll
    for (int d = 0; d < kHcMaxMult; ++d)
      *reinterpret_cast<float4*>(&xs[rr][d][c]) = make_float4(out[d][0], out[d][1], out[d][2], out[d][3]);
  }
  __syncthreads();
  // ---- partial mixes: warp w owns projections w, w+8, w+16
  float dot[3][kHcRowsPerBlock];
  float sq[kHcRowsPerBlock];
#pragma unroll
  for (int j = 0; j < 3; ++j)
#pragma unroll
    for (int rr = 0; rr < kHcRowsPerBlock; ++rr) dot[j][rr] = 0.f;
#pragma unroll
  for (int rr = 0; rr < kHcRowsPerBlock; ++rr) sq[rr] = 0.f;
#pragma unroll 8
  for (int idx = lane; idx < kHcMaxMult * kHcSlice; idx += 32) {
    const int d = idx / kHcSlice, c = idx % kHcSlice;
    float f[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) f[j] = fs[(warp + 8 * j) * (kHcMaxMult * kHcSlice) + idx];
#pragma unroll
    for (int rr = 0; rr < kHcRowsPerBlock; ++rr) {
      const float x = xs[rr][d][c];
#pragma unroll
      for (int j = 0; j < 3; ++j) dot[j][rr] = fmaf(x, f[j], dot[j][rr]);
      if (warp == 0) sq[rr] = fmaf(x, x, sq[rr]);
    }
  }
#pragma unroll
  for (int rr = 0; rr < kHcRowsPerBlock; ++rr) {
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const float v = warp_sum(dot[j][rr]);
      if (lane == 0 && r0 + rr < rows)
        partial[(1ll * blockIdx.x * rows + r0 + rr) * kHcPartialStride + warp + 8 * j] = v;
    }
    if (warp == 0) {
      const float v = warp_sum(sq[rr]);
      if (lane == 0 && r0 + rr < rows) partial[(1ll * blockIdx.x * rows + r0 + rr) * kHcPartialStride + kHcProj] = v;
    }
  }
  }   // row groups of this block
}

// Expand alone, for passes whose mixes projection runs as a GEMM afterwards: one block per row walks the row's H
// columns in groups of eight (16-byte stream loads and stores, two 16-byte loads per partial plane), with the row's
// 4 + 16 mixing coefficients in registers, and leaves the sum of squares of the new streams in
// partial[row * kHcPartialStride + kHcProj] (one slice).  parts.n_ranks == 0: the streams stay as they are and only the
// sum of squares is produced.
// With `xn` the block also collapses the new streams with the incoming weights `pre_in` and normalises the row
// (what hc_finish does from a second read of the streams): x = sum_s pre_in[s] * streams'[s], xn = x * rsqrt(mean x^2 +
// eps) * norm_w, and the drafter's tap mean if asked for.  The collapsed values of a thread's groups stay in registers
// across the block-wide sum (H <= 6144).
__global__ void __launch_bounds__(256)
hc_expand_kernel(const __nv_bfloat16* streams_in, __nv_bfloat16* streams_out, PartList parts,
                 const float* __restrict__ post, const float* __restrict__ comb, float* __restrict__ partial, int rows,
                 int H, const uint32_t* const* __restrict__ wait_flags, const uint32_t* __restrict__ wait_epoch,
                 int* status, const float* __restrict__ pre_in, const float* __restrict__ norm_w,
                 __nv_bfloat16* __restrict__ xn, float* __restrict__ tap_mean, float norm_eps) {
  __shared__ float warp_sq[8];
  __shared__ float warp_xsq[8];
  __shared__ float inv_rms;
  constexpr int kMaxItems = 3;
  float keep[kMaxItems][8];
  float x_sq = 0.f;
  float p_in[kHcMaxMult] = {0.f, 0.f, 0.f, 0.f};
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  pdl_wait();
  if (wait_flags != nullptr && parts.n_ranks > 1) {
    if (tid < parts.n_ranks) flag_wait_ge(wait_flags[tid], *wait_epoch, status, 400 + tid);
    __syncthreads();
  }
  const bool expand = parts.n_ranks > 0;
  float cm[16], pw[4];
  if (expand) {
#pragma unroll
    for (int q = 0; q < 16; ++q) cm[q] = comb[r * 16 + q];
#pragma unroll
    for (int q = 0; q < 4; ++q) pw[q] = post[r * 4 + q];
  }
  if (xn != nullptr) {
#pragma unroll
    for (int q = 0; q < kHcMaxMult; ++q) p_in[q] = pre_in[r * 4 + q];
  }
  const int n_sp = parts.n_splits, total = parts.n_ranks * n_sp;
  float sq = 0.f;
#pragma unroll
  for (int n = 0; n < kMaxItems; ++n) {
    const int g = tid + 256 * n;
    if (g >= H / 8) continue;
    const int c = g * 8;
    uint4 raw[kHcMaxMult];
#pragma unroll
    for (int s = 0; s < kHcMaxMult; ++s)
      raw[s] = *reinterpret_cast<const uint4*>(streams_in + (1ll * r * kHcMaxMult + s) * H + c);
    float s_in[kHcMaxMult][8];
#pragma unroll
    for (int s = 0; s < kHcMaxMult; ++s) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[s]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 v = __bfloat1622float2(h[q]);
        s_in[s][2 * q] = v.x;
        s_in[s][2 * q + 1] = v.y;
      }
    }
    float out[kHcMaxMult][8];
    if (!expand) {
#pragma unroll
      for (int s = 0; s < kHcMaxMult; ++s)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          out[s][j] = s_in[s][j];
          sq = fmaf(s_in[s][j], s_in[s][j], sq);
        }
    } else {
    float sub[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // rank-major, split-minor order; four planes (eight 16-byte loads) in flight before the first add
    for (int j0 = 0; j0 < total; j0 += 4) {
      float4 v[4][2];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u;
        v[u][0] = v[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < total) {
          const int k = j / n_sp, sp = j - k * n_sp;
          const float4* src = reinterpret_cast<const float4*>(parts.base[k] + sp * parts.split_stride + 1ll * r * H + c);
          v[u][0] = __ldcg(src);
          v[u][1] = __ldcg(src + 1);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        sub[0] += v[u][0].x; sub[1] += v[u][0].y; sub[2] += v[u][0].z; sub[3] += v[u][0].w;
        sub[4] += v[u][1].x; sub[5] += v[u][1].y; sub[6] += v[u][1].z; sub[7] += v[u][1].w;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sb = bf16_round(sub[j]);
#pragma unroll
      for (int d = 0; d < kHcMaxMult; ++d) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < kHcMaxMult; ++s) acc = fmaf(cm[s * 4 + d], s_in[s][j], acc);
        out[d][j] = bf16_round(fmaf(pw[d], sb, acc));
        sq = fmaf(out[d][j], out[d][j], sq);
      }
    }
#pragma unroll
    for (int d = 0; d < kHcMaxMult; ++d) {
      uint4 w;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(out[d][2 * q], out[d][2 * q + 1]);
      *reinterpret_cast<uint4*>(streams_out + (1ll * r * kHcMaxMult + d) * H + c) = w;
    }
    }   // expand
    if (xn != nullptr) {
      // same arithmetic and summation order as hc_finish, so that both forms give identical rows
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float x = bf16_round(fmaf(p_in[3], out[3][2 * q], fmaf(p_in[2], out[2][2 * q],
                                   fmaf(p_in[1], out[1][2 * q], p_in[0] * out[0][2 * q]))));
        const float y = bf16_round(fmaf(p_in[3], out[3][2 * q + 1], fmaf(p_in[2], out[2][2 * q + 1],
                                   fmaf(p_in[1], out[1][2 * q + 1], p_in[0] * out[0][2 * q + 1]))));
        keep[n][2 * q] = x;
        keep[n][2 * q + 1] = y;
        x_sq = fmaf(x, x, fmaf(y, y, x_sq));
      }
      if (tap_mean != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          tap_mean[1ll * r * H + c + j] = 0.25f * (out[0][j] + out[1][j] + out[2][j] + out[3][j]);
      }
    }
  }
  sq = warp_sum(sq);
  x_sq = warp_sum(x_sq);
  if (lane == 0) {
    warp_sq[warp] = sq;
    warp_xsq[warp] = x_sq;
  }
  __syncthreads();
  if (tid == 0) {
    float t = 0.f, u = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { t += warp_sq[w]; u += warp_xsq[w]; }
    partial[1ll * r * kHcPartialStride + kHcProj] = t;
    inv_rms = rsqrtf(u / H + norm_eps);
  }
  if (xn == nullptr) return;
  __syncthreads();
  const float inv = inv_rms;
#pragma unroll
  for (int n = 0; n < kMaxItems; ++n) {
    const int g = tid + 256 * n;
    if (g >= H / 8) continue;
    float y[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) y[q] = bf16_round(keep[n][q] * inv * (norm_w != nullptr ? norm_w[8 * g + q] : 1.f));
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(y[2 * q], y[2 * q + 1]);
    *reinterpret_cast<uint4*>(xn + 1ll * r * H + 8 * g) = o;
  }
}

// One block per row.  Produces next_pre/post/comb from the slice partials, then the collapsed,
// normalised row.  `norm_w` may be null (no weight).  When `xq` is given the normalised row is also emitted
// as E4M3 with one power-of-two scale per 128 columns, written in the MX GEMM's scale-atom layout.
__global__ void __launch_bounds__(256)
hc_finish_kernel(const float* __restrict__ partial, int n_slices, const float* __restrict__ scale,
                 const float* __restrict__ base, const float* __restrict__ pre_in,
                 const __nv_bfloat16* __restrict__ streams, const float* __restrict__ norm_w,
                 float* __restrict__ next_pre, float* __restrict__ post, float* __restrict__ comb,
                 __nv_bfloat16* __restrict__ xn, float* __restrict__ tap_mean, uint8_t* __restrict__ xq,
                 uint8_t* __restrict__ xq_sf, int rows, int H, int iters, float hc_eps, float norm_eps,
                 const float* __restrict__ mix_planes, int mix_splits, long long mix_split_stride, int mix_ld) {
  __shared__ float proj[kHcProj + 1];
  __shared__ float warp_part[8];
  __shared__ float inv_rms;
  const int r = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  // ---- slice partials: warp w reduces values w, w+8, w+16 (+24); fixed shuffle tree -> deterministic
  for (int j = warp; j <= kHcProj; j += 8) {
    float acc = 0.f;
    if (mix_planes != nullptr && j < kHcProj) {
      // tensor-core projection: split-K planes [split][rows][mix_ld], columns j (high part) and 24 + j (low part)
      for (int s = lane; s < mix_splits; s += 32) {
        const float* p = mix_planes + s * mix_split_stride + 1ll * r * mix_ld;
        acc += p[j] + p[kHcProj + j];
      }
    } else {
      for (int s = lane; s < n_slices; s += 32) acc += partial[(1ll * s * rows + r) * kHcPartialStride + j];
    }
    acc = warp_sum(acc);
    if (lane == 0) proj[j] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    const float inv = rsqrtf(proj[kHcProj] / (4.0f * H) + norm_eps);
    if (lane < 4) {
      const float a = fmaf(proj[lane] * inv, scale[0], base[lane]);
      const float b = fmaf(proj[lane + 4] * inv, scale[1], base[lane + 4]);
      next_pre[r * 4 + lane] = 1.0f / (1.0f + __expf(-a)) + hc_eps;
      post[r * 4 + lane] = 2.0f / (1.0f + __expf(-b));
    }
    // comb: lane = s*4 + d for lanes < 16
    float v = lane < 16 ? fmaf(proj[8 + lane] * inv, scale[2], base[8 + lane]) : 0.f;
    float mx = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    v = __expf(v - mx);
    float sum = v + __shfl_xor_sync(0xffffffffu, v, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    v = v / sum + hc_eps;
    sum = v + __shfl_xor_sync(0xffffffffu, v, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    v /= sum + hc_eps;
    for (int it = 1; it < iters; ++it) {
      sum = v + __shfl_xor_sync(0xffffffffu, v, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      v /= sum + hc_eps;
      sum = v + __shfl_xor_sync(0xffffffffu, v, 4);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      v /= sum + hc_eps;
    }
    if (lane < 16) comb[r * 16 + lane] = v;
  }
  if (xn == nullptr) return;        // the expand kernel already collapsed and normalised the row
  // ---- collapse with the incoming pre + RMSNorm; each thread owns up to 3 groups of 8 columns
  const float p0 = pre_in[r * 4 + 0], p1 = pre_in[r * 4 + 1], p2 = pre_in[r * 4 + 2], p3 = pre_in[r * 4 + 3];
  const __nv_bfloat16* s0 = streams + 1ll * r * 4 * H;
  constexpr int kMaxItems = 3;               // H <= 256 * 3 * 8 = 6144
  float keep[kMaxItems][8];
  float local_sq = 0.f;
  const int n_items = H / 8;
#pragma unroll
  for (int n = 0; n < kMaxItems; ++n) {
    const int i = tid + 256 * n;
    if (i < n_items) {
      uint4 raw[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) raw[s] = *reinterpret_cast<const uint4*>(s0 + 1ll * s * H + 8 * i);
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&raw[0]);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&raw[1]);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[2]);
      const __nv_bfloat162* h3 = reinterpret_cast<const __nv_bfloat162*>(&raw[3]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __bfloat1622float2(h0[q]), b = __bfloat1622float2(h1[q]);
        const float2 c = __bfloat1622float2(h2[q]), d = __bfloat1622float2(h3[q]);
        const float x = bf16_round(fmaf(p3, d.x, fmaf(p2, c.x, fmaf(p1, b.x, p0 * a.x))));
        const float y = bf16_round(fmaf(p3, d.y, fmaf(p2, c.y, fmaf(p1, b.y, p0 * a.y))));
        keep[n][2 * q] = x;
        keep[n][2 * q + 1] = y;
        local_sq = fmaf(x, x, fmaf(y, y, local_sq));
        if (tap_mean != nullptr) {
          tap_mean[1ll * r * H + 8 * i + 2 * q] = 0.25f * (a.x + b.x + c.x + d.x);
          tap_mean[1ll * r * H + 8 * i + 2 * q + 1] = 0.25f * (a.y + b.y + c.y + d.y);
        }
      }
    }
  }
  local_sq = warp_sum(local_sq);
  if (lane == 0) warp_part[warp] = local_sq;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += warp_part[w];
    inv_rms = rsqrtf(t / H + norm_eps);
  }
  __syncthreads();
  const float inv = inv_rms;
#pragma unroll
  for (int n = 0; n < kMaxItems; ++n) {
    const int i = tid + 256 * n;
    const bool live = i < n_items;
    float y[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float w = (live && norm_w != nullptr) ? norm_w[8 * i + q] : 1.f;
      y[q] = live ? bf16_round(keep[n][q] * inv * w) : 0.f;
    }
    if (live) {
      uint4 o;
      __nv_bfloat162 t0 = __floats2bfloat162_rn(y[0], y[1]), t1 = __floats2bfloat162_rn(y[2], y[3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(y[4], y[5]), t3 = __floats2bfloat162_rn(y[6], y[7]);
      o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
      o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
      *reinterpret_cast<uint4*>(xn + 1ll * r * H + 8 * i) = o;
    }
    if (xq != nullptr) {
      // 16 consecutive lanes hold one 128-column group (H is a multiple of 128, so groups never straddle `live`)
      float amax = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(y[q]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
      float sc = fmaxf(amax * (1.0f / 448.0f), 1.17549435e-38f);
      uint32_t bits = __float_as_uint(sc);
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
        *reinterpret_cast<uint2*>(xq + 1ll * r * H + 8 * i) = o;
        if ((i & 15) == 0) {
          const int kc = i / 16;
          uint8_t* atom = xq_sf + (1ll * (r / 128) * (H / 128) + kc) * 512;
          *reinterpret_cast<uint32_t*>(atom + (r % 32) * 16 + ((r / 32) % 4) * 4) = e * 0x01010101u;
        }
      }
    }
  }
}

// Coefficients alone, one warp per row: the 24 projections come from the GEMM's split-K planes (high + low part per
// split, splits in order), the sum of squares from the expand kernel; the rest is hc_finish's first phase.
__global__ void __launch_bounds__(256)
hc_mixes_kernel(const float* __restrict__ partial, const float* __restrict__ scale, const float* __restrict__ base,
                float* __restrict__ next_pre, float* __restrict__ post, float* __restrict__ comb, int rows, int H,
                int iters, float hc_eps, float norm_eps, const float* __restrict__ mix_planes, int mix_splits,
                long long mix_split_stride, int mix_ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  float acc = 0.f;
  if (lane < kHcProj) {
    for (int s = 0; s < mix_splits; ++s) {
      const float* p = mix_planes + s * mix_split_stride + 1ll * r * mix_ld;
      acc += p[lane] + p[kHcProj + lane];
    }
  }
  const float inv = rsqrtf(partial[1ll * r * kHcPartialStride + kHcProj] / (4.0f * H) + norm_eps);
  const float proj = acc * inv;
  const float p_post = __shfl_sync(0xffffffffu, proj, (lane + 4) & 31);
  const float p_comb = __shfl_sync(0xffffffffu, proj, (lane + 8) & 31);
  if (lane < 4) {
    const float a = fmaf(proj, scale[0], base[lane]);
    const float b = fmaf(p_post, scale[1], base[lane + 4]);
    next_pre[r * 4 + lane] = 1.0f / (1.0f + __expf(-a)) + hc_eps;
    post[r * 4 + lane] = 2.0f / (1.0f + __expf(-b));
  }
  // comb: lane = s*4 + d for lanes < 16
  float v = lane < 16 ? fmaf(p_comb, scale[2], base[8 + lane]) : 0.f;
  float mx = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  v = __expf(v - mx);
  float sum = v + __shfl_xor_sync(0xffffffffu, v, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  v = v / sum + hc_eps;
  sum = v + __shfl_xor_sync(0xffffffffu, v, 4);
  sum += __shfl_xor_sync(0xffffffffu, sum, 8);
  v /= sum + hc_eps;
  for (int it = 1; it < iters; ++it) {
    sum = v + __shfl_xor_sync(0xffffffffu, v, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    v /= sum + hc_eps;
    sum = v + __shfl_xor_sync(0xffffffffu, v, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    v /= sum + hc_eps;
  }
  if (lane < 16) comb[r * 16 + lane] = v;
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_embed_streams(const int* tokens, const void* embed, void* streams, float* pre, int rows, int H,
                                  int mult, int vocab, void* stream) {
  if (rows <= 0 || H % 8 != 0 || mult != kHcMaxMult) return cudaErrorInvalidValue;
  return launch_pdl(embed_streams_kernel, dim3(rows), dim3(128), 0, static_cast<cudaStream_t>(stream), tokens,
                    static_cast<const __nv_bfloat16*>(embed), static_cast<__nv_bfloat16*>(streams), pre, rows, H,
                    mult, vocab);
}

extern "C" int ds41_hc_post_mix(const void* streams_in, void* streams_out, const float* const* part_bases,
                                int n_ranks, int n_splits, long long split_stride, const float* post,
                                const float* comb, const float* fn, float* partial, int rows, int H,
                                const uint32_t* const* wait_flags, const uint32_t* wait_epoch, int* status,
                                const float* pre_in, const float* norm_w, void* xn, float* tap_mean, float norm_eps,
                                void* stream) {
  if (rows <= 0 || H % kHcSlice != 0 || n_ranks < 0 || n_ranks > 8) return cudaErrorInvalidValue;
  if (xn != nullptr && (fn != nullptr || pre_in == nullptr || H > 256 * 3 * 8)) return cudaErrorInvalidValue;
  PartList parts{};
  parts.n_ranks = n_ranks;
  parts.n_splits = n_splits;
  parts.split_stride = split_stride;
  for (int i = 0; i < n_ranks; ++i) parts.base[i] = part_bases[i];
  // rows per block: as many eight-row groups as still leave about two blocks per SM
  const int slices = H / kHcSlice;
  int rpb = rows * slices / (2 * 148) / kHcRowsPerBlock * kHcRowsPerBlock;
  rpb = rpb < kHcRowsPerBlock ? kHcRowsPerBlock : (rpb > 64 ? 64 : rpb);
  if (fn == nullptr)      // expand only; the sum of squares of row r lands in partial[r * 25 + 24] (one slice)
    return launch_pdl(hc_expand_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                      static_cast<const __nv_bfloat16*>(streams_in), static_cast<__nv_bfloat16*>(streams_out), parts,
                      post, comb, partial, rows, H, wait_flags, wait_epoch, status, pre_in, norm_w,
                      static_cast<__nv_bfloat16*>(xn), tap_mean, norm_eps);
  constexpr size_t kSmem = sizeof(float) * (kHcRowsPerBlock * kHcMaxMult * kHcSlice + kHcProj * kHcMaxMult * kHcSlice);
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(hc_post_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSmem));
    if (e != cudaSuccess) return e;
    configured[dev].store(true, std::memory_order_release);
  }
  dim3 grid(slices, (rows + rpb - 1) / rpb);
  return launch_pdl(hc_post_mix_kernel, grid, dim3(256), kSmem, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(streams_in), static_cast<__nv_bfloat16*>(streams_out), parts,
                    post, comb, fn, partial, rows, H, wait_flags, wait_epoch, status, rpb);
}

extern "C" int ds41_hc_finish(const float* partial, int n_slices, const float* scale, const float* base,
                              const float* pre_in, const void* streams, const float* norm_w, float* next_pre,
                              float* post, float* comb, void* xn, float* tap_mean, void* xq, void* xq_sf, int rows,
                              int H, int iters, float hc_eps, float norm_eps, const float* mix_planes, int mix_splits,
                              long long mix_split_stride, int mix_ld, void* stream) {
  if (rows <= 0 || H % 8 != 0 || H > 256 * 3 * 8 || (xq != nullptr && (H % 128 != 0 || xq_sf == nullptr)) ||
      (mix_planes != nullptr && (mix_splits <= 0 || mix_ld < 2 * kHcProj)))
    return cudaErrorInvalidValue;
  if (xn == nullptr && mix_planes != nullptr)           // coefficients only: one warp per row
    return launch_pdl(hc_mixes_kernel, dim3((rows + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), partial,
                      scale, base, next_pre, post, comb, rows, H, iters, hc_eps, norm_eps, mix_planes, mix_splits,
                      mix_split_stride, mix_ld);
  return launch_pdl(hc_finish_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), partial, n_slices,
                    scale, base, pre_in, static_cast<const __nv_bfloat16*>(streams), norm_w, next_pre, post, comb,
                    static_cast<__nv_bfloat16*>(xn), tap_mean, static_cast<uint8_t*>(xq),
                    static_cast<uint8_t*>(xq_sf), rows, H, iters, hc_eps, norm_eps, mix_planes, mix_splits,
                    mix_split_stride, mix_ld);
}
