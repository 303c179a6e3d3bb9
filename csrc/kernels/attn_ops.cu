// Attention-side elementwise / cache kernels:
//   qkv_post   : reduce the split-K planes of the fused [wq_a | wkv | compressor | index-weight] projection,
//                RMSNorm(q latent), RMSNorm+RoPE(kv) and the position-indexed window-ring write
//   compress   : softmax-gated pair pooling (ratio 2) or pass-through (ratio 1), RMSNorm, index-key
//                projection + norm + RoPE, RoPE of the latent, paged pool writes
// Behaviour follows the reference's native/cuda/kernels/v41_attention_ops.cu:24-68 (norm/RoPE),
// v41_kv.cu:48-61 (scatter store) and v41_compressor.cu:69-108 (pool); the cache protocol differs on
// purpose: every cache row is addressed by token position (ring slot = pos % ring_rows, compressed row =
// pos / ratio), so rows written for drafts that are later rejected are simply rewritten when the position
// is processed again and never read before that - no proposal overlay or commit copy is needed.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

// FP8 cache row: D e4m3 bytes, then D/32 UE8M0 scale bytes (scale = ceil_pow2(amax / 448) per 32 elements), padded to a
// multiple of 16 bytes.  The calling thread holds elements (2i, 2i+1); 16 consecutive lanes form one 32-element group.
// Every lane of the warp must call (inactive lanes pass zeros and active = false).
__device__ __forceinline__ void store_kv_fp8_pair(uint8_t* row, int D, int i, float a, float b, bool active) {
  float amax = fmaxf(fabsf(a), fabsf(b));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
  if (!active) return;
  const uint32_t e = ue8m0_ceil_exp(amax * (1.0f / 448.0f));
  const float inv = __uint_as_float((254u - e) << 23);
  const __nv_fp8x2_e4m3 q(make_float2(a * inv, b * inv));
  *reinterpret_cast<uint16_t*>(row + 2 * i) = *reinterpret_cast<const uint16_t*>(&q);
  if ((i & 15) == 0) row[D + (i >> 4)] = static_cast<uint8_t>(e);
}


// Compressed-cache row in FP4: D/2 bytes of e2m1 pairs (even element in the low nibble), then D/16 E4M3 scales, one per
// 16 values: scale = e4m3(max(amax, 6 * 2^-9) / 6), code = e2m1(value / scale).  Thread i owns elements 2i, 2i+1; the
// eight threads of a 16-value group share the scale.  All lanes of a warp call it (shuffles); `active` gates the stores.
// Format parity: native/cuda/kernels/v41_kv.cu:29-39 of the reference.
__device__ __forceinline__ void store_kv_fp4_pair(uint8_t* row, int D, int i, float a, float b, bool active) {
  float amax = fmaxf(fabsf(a), fabsf(b));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  if (!active) return;
  amax = fmaxf(amax, 6.0f * 0.001953125f);
  const __nv_fp8_e4m3 sc(__fdiv_rn(amax, 6.0f));
  const float scf = static_cast<float>(sc);
  const uint32_t ca = e2m1_code(__fdiv_rn(a, scf)), cb = e2m1_code(__fdiv_rn(b, scf));
  row[i] = static_cast<uint8_t>(ca | (cb << 4));
  if ((i & 7) == 0) row[D / 2 + (i >> 3)] = *reinterpret_cast<const uint8_t*>(&sc);
}

__device__ __forceinline__ void rope_cs(int pos, float inv_freq, float* c, float* s) {
  // reduce the angle in double so positions up to 2^20 keep fp32-accurate sin/cos
  const double a = static_cast<double>(pos) * static_cast<double>(inv_freq);
  const double two_pi = 6.283185307179586476925286766559;
  const double red = a - floor(a * 0.15915494309189533576888376337251) * two_pi;
  sincosf(static_cast<float>(red), s, c);
}

__device__ __forceinline__ float block_sum_256(float v, float* scratch /*[8]*/) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += scratch[w];
  return t;
}

struct QkvPostParams {
  const float* planes;      // [splits][rows][ntot]
  int splits, rows, ntot;
  int Q, D, rope_dim;
  int extra_f32;            // columns after q|kv copied as fp32 (compressor kv/gate, index weights)
  int index_heads;          // last `index_heads` columns of the extras are scaled by index_scale
  float index_scale;
  const float* q_norm_w;
  const float* kv_norm_w;
  const float* inv_freq;    // [rope_dim/2]
  const int* row_pos;
  const int* row_slot;
  __nv_bfloat16* q_lat;     // [rows][Q]
  __nv_bfloat16* win;       // [slots][ring][D] bf16, or FP8 rows of kv_row_bytes bytes (see store_kv_fp8_pair)
  int ring;
  int kv_row_bytes;         // 0: bf16 rows
  float* extras;            // [rows][extra_f32]
  float eps;
};

// grid (rows, 2): block y == 0 normalises the q latent, y == 1 handles kv (norm + RoPE + ring write) and extras.
__global__ void __launch_bounds__(256) qkv_post_kernel(QkvPostParams p) {
  __shared__ float scratch[8];
  const int r = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const long long plane = 1ll * p.rows * p.ntot;
  const float* row0 = p.planes + 1ll * r * p.ntot;
  if (blockIdx.y == 0) {
    // ---- q latent (Q <= 2048: up to 8 columns per thread, all split loads issued together)
    float vals[8];
    float sq = 0.f;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int c = tid + 256 * n;
      float a = 0.f;
      if (c < p.Q) {
#pragma unroll 4
        for (int s = 0; s < p.splits; ++s) a += row0[s * plane + c];
        a = bf16_round(a);
      }
      vals[n] = a;
      sq = fmaf(a, a, sq);
    }
    const float tot = block_sum_256(sq, scratch);
    const float inv = rsqrtf(tot / p.Q + p.eps);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int c = tid + 256 * n;
      if (c < p.Q) p.q_lat[1ll * r * p.Q + c] = __float2bfloat16_rn(vals[n] * inv * p.q_norm_w[c]);
    }
    return;
  }
  // ---- kv: thread handles adjacent pairs so RoPE stays in-thread (D <= 2048)
  float2 kvv[4];
  float sq = 0.f;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int i = tid + 256 * n;
    float a = 0.f, b = 0.f;
    if (i < p.D / 2) {
#pragma unroll 4
      for (int s = 0; s < p.splits; ++s) {
        const float2 v = *reinterpret_cast<const float2*>(row0 + s * plane + p.Q + 2 * i);
        a += v.x;
        b += v.y;
      }
      a = bf16_round(a);
      b = bf16_round(b);
    }
    kvv[n] = make_float2(a, b);
    sq = fmaf(a, a, fmaf(b, b, sq));
  }
  const float tot = block_sum_256(sq, scratch);
  const float inv = rsqrtf(tot / p.D + p.eps);
  const int pos = p.row_pos[r];
  const int slot = p.row_slot[r];
  const long long ring_row = 1ll * slot * p.ring + (pos % p.ring);
  __nv_bfloat16* dst = p.win + ring_row * p.D;
  uint8_t* dst8 = reinterpret_cast<uint8_t*>(p.win) + ring_row * p.kv_row_bytes;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int i = tid + 256 * n;
    if (256 * n >= p.D / 2) break;                      // uniform over the block
    const bool active = i < p.D / 2;
    float a = 0.f, b = 0.f;
    if (active) {
      a = bf16_round(kvv[n].x * inv * p.kv_norm_w[2 * i]);
      b = bf16_round(kvv[n].y * inv * p.kv_norm_w[2 * i + 1]);
      const int t = 2 * i - (p.D - p.rope_dim);
      if (t >= 0) {
        float c, s;
        rope_cs(pos, p.inv_freq[t / 2], &c, &s);
        const float ra = a * c - b * s;
        const float rb = b * c + a * s;
        a = ra;
        b = rb;
      }
    }
    if (p.kv_row_bytes > 0) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);      // the cache holds the FP8 image of the bf16 row
      store_kv_fp8_pair(dst8, p.D, i, __low2float(h), __high2float(h), active && slot >= 0);
    } else if (active && slot >= 0) {
      reinterpret_cast<__nv_bfloat162*>(dst)[i] = __floats2bfloat162_rn(a, b);
    }
  }
  // ---- extras (fp32 pass-through; index weights scaled)
  for (int c = tid; c < p.extra_f32; c += 256) {
    float a = 0.f;
    for (int s = 0; s < p.splits; ++s) a += row0[s * plane + p.Q + p.D + c];
    if (c >= p.extra_f32 - p.index_heads) a *= p.index_scale;
    p.extras[1ll * r * p.extra_f32 + c] = a;
  }
}

struct CompressParams {
  const float* extras;       // [rows][extra_stride]: ckv at col 0, cgate at col D (ratio 2)
  int extra_stride;
  int rows, D, ID, rope_dim, ratio;
  const int* row_pos;
  const int* row_slot;
  float* pending;            // [slots][4][2*D] fp32: (kv, gate) of recent even positions, by (pos/2)&3
  const float* comp_norm_w;  // [D]
  const __nv_bfloat16* wk;   // [ID][D]
  const float* k_norm_w;     // [ID]
  const float* inv_freq;     // [rope_dim/2]
  const float* inv_freq_idx; // [ID/4]
  const int* page_table;     // [slots][max_pages]
  int max_pages, page_rows;
  __nv_bfloat16* comp_pool;  // [pool_rows][D] bf16, FP8 rows of kv_row_bytes bytes, or FP4 rows of -kv_row_bytes bytes
  int kv_row_bytes;
  __nv_bfloat16* idx_pool;   // [pool_rows][ID] bf16, or FP4 rows of idx_row_bytes bytes (ID/2 E2M1 bytes + ID/32 UE8M0)
  float eps;
  int idx_row_bytes;
};

// One block (256 threads) per row.  D <= 1024, ID <= 256.
__global__ void __launch_bounds__(256) compress_kernel(CompressParams p) {
  __shared__ float scratch[8];
  __shared__ float latent[1024];
  __shared__ float ikey[256];
  const int r = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.row_pos[r], slot = p.row_slot[r];
  if (slot < 0) return;
  const float* cur = p.extras + 1ll * r * p.extra_stride;
  int first_pos = pos;
  if (p.ratio == 2) {
    float* pend = p.pending + (1ll * slot * 4 + ((pos >> 1) & 3)) * 2 * p.D;
    if ((pos & 1) == 0) {
      // The carry has four places per request, indexed by (pos / 2) & 3, so that a rejected speculative row leaves
      // the carry of the accepted ones intact.  In a pass longer than 8 positions two even rows 8 apart share a
      // place: only the later one may write it (its block can run before or after the earlier row's block).
      const bool later_writer = r + 8 < p.rows && p.row_slot[r + 8] == slot && p.row_pos[r + 8] == pos + 8;
      if (!later_writer)
        for (int c = tid; c < 2 * p.D; c += 256) pend[c] = cur[c];
      return;
    }
    const float* prev = pend;
    if (r > 0 && p.row_slot[r - 1] == slot && p.row_pos[r - 1] == pos - 1) prev = p.extras + 1ll * (r - 1) * p.extra_stride;
    for (int c = tid; c < p.D; c += 256) {
      const float a = prev[p.D + c], b = cur[p.D + c], mx = fmaxf(a, b);
      const float ea = __expf(a - mx), eb = __expf(b - mx), sum = ea + eb;
      latent[c] = bf16_round(prev[c] * (ea / sum) + cur[c] * (eb / sum));
    }
    first_pos = pos - 1;
  } else {
    for (int c = tid; c < p.D; c += 256) latent[c] = bf16_round(cur[c]);
  }
  __syncthreads();
  float sq = 0.f;
  for (int c = tid; c < p.D; c += 256) sq = fmaf(latent[c], latent[c], sq);
  float tot = block_sum_256(sq, scratch);
  float inv = rsqrtf(tot / p.D + p.eps);
  for (int c = tid; c < p.D; c += 256) latent[c] = bf16_round(latent[c] * inv * p.comp_norm_w[c]);
  __syncthreads();
  // ---- index key: ik[j] = sum_d wk[j][d] * latent[d]; one warp per output, 8 warps
  const int warp = tid >> 5, lane = tid & 31;
  for (int j = warp; j < p.ID; j += 8) {
    const __nv_bfloat16* w = p.wk + 1ll * j * p.D;
    float acc = 0.f;
    for (int d = lane * 2; d < p.D; d += 64) {
      const float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + d));
      acc = fmaf(wv.x, latent[d], fmaf(wv.y, latent[d + 1], acc));
    }
    acc = warp_sum(acc);
    if (lane == 0) ikey[j] = bf16_round(acc);
  }
  __syncthreads();
  sq = 0.f;
  for (int c = tid; c < p.ID; c += 256) sq = fmaf(ikey[c], ikey[c], sq);
  tot = block_sum_256(sq, scratch);
  inv = rsqrtf(tot / p.ID + p.eps);
  const int crow = pos / p.ratio;
  const int page = p.page_table[1ll * slot * p.max_pages + crow / p.page_rows];
  if (page < 0) return;
  const long long phys = 1ll * page * p.page_rows + crow % p.page_rows;
  const int idx_rope = p.ID / 2;
  for (int i = tid; i < p.ID / 2; i += 256) {
    const unsigned lanes = __activemask();          // whole 16-lane groups: ID / 2 is a multiple of 16
    float a = bf16_round(ikey[2 * i] * inv * p.k_norm_w[2 * i]);
    float b = bf16_round(ikey[2 * i + 1] * inv * p.k_norm_w[2 * i + 1]);
    const int t = 2 * i - (p.ID - idx_rope);
    if (t >= 0) {
      float c, s;
      rope_cs(first_pos, p.inv_freq_idx[t / 2], &c, &s);
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    if (p.idx_row_bytes == 0) {
      reinterpret_cast<__nv_bfloat162*>(p.idx_pool + phys * p.ID)[i] = __floats2bfloat162_rn(a, b);
    } else {
      // FP4 key row: the 16 threads of a 32-value group share one scale (ID / 2 is a multiple of 16, so the groups
      // are whole in every active warp)
      uint8_t* row = reinterpret_cast<uint8_t*>(p.idx_pool) + phys * p.idx_row_bytes;
      uint32_t e;
      const uint32_t byte = fp4_group_pack(bf16_round(a), bf16_round(b), &e, lanes);
      row[i] = static_cast<uint8_t>(byte);
      if ((i & 15) == 0) row[p.ID / 2 + (i >> 4)] = static_cast<uint8_t>(e);
    }
  }
  for (int i0 = 0; i0 < p.D / 2; i0 += 256) {
    const int i = i0 + tid;
    const bool active = i < p.D / 2;
    float a = 0.f, b = 0.f;
    if (active) {
      a = latent[2 * i];
      b = latent[2 * i + 1];
      const int t = 2 * i - (p.D - p.rope_dim);
      if (t >= 0) {
        float c, s;
        rope_cs(first_pos, p.inv_freq[t / 2], &c, &s);
        const float ra = a * c - b * s, rb = b * c + a * s;
        a = ra;
        b = rb;
      }
    }
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    if (p.kv_row_bytes < 0)        // FP4 rows of -kv_row_bytes bytes
      store_kv_fp4_pair(reinterpret_cast<uint8_t*>(p.comp_pool) + phys * (-p.kv_row_bytes), p.D, i, __low2float(h),
                        __high2float(h), active);
    else if (p.kv_row_bytes > 0)
      store_kv_fp8_pair(reinterpret_cast<uint8_t*>(p.comp_pool) + phys * p.kv_row_bytes, p.D, i, __low2float(h),
                        __high2float(h), active);
    else if (active)
      reinterpret_cast<__nv_bfloat162*>(p.comp_pool + phys * p.D)[i] = h;
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_qkv_post(const float* planes, int splits, int rows, int ntot, int Q, int D, int rope_dim,
                             int extra_f32, int index_heads, float index_scale, const float* q_norm_w,
                             const float* kv_norm_w, const float* inv_freq, const int* row_pos, const int* row_slot,
                             void* q_lat, void* win, int ring, float* extras, float eps, int kv_row_bytes,
                             void* stream) {
  if (rows <= 0 || Q > 2048 || D > 2048 || (D & 1) || (rope_dim & 1) || Q + D + extra_f32 > ntot)
    return cudaErrorInvalidValue;
  if (kv_row_bytes != 0 && (kv_row_bytes < D + D / 32 || (D & 31) || (kv_row_bytes & 15))) return cudaErrorInvalidValue;
  QkvPostParams p{planes, splits, rows, ntot, Q, D, rope_dim, extra_f32, index_heads, index_scale, q_norm_w,
                  kv_norm_w, inv_freq, row_pos, row_slot, static_cast<__nv_bfloat16*>(q_lat),
                  static_cast<__nv_bfloat16*>(win), ring, kv_row_bytes, extras, eps};
  if ((Q + D) & 1) return cudaErrorInvalidValue;   // kv columns are read as aligned float2
  return launch_pdl(qkv_post_kernel, dim3(rows, 2), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_compress(const float* extras, int extra_stride, int rows, int D, int ID, int rope_dim, int ratio,
                             const int* row_pos, const int* row_slot, float* pending, const float* comp_norm_w,
                             const void* wk, const float* k_norm_w, const float* inv_freq, const float* inv_freq_idx,
                             const int* page_table, int max_pages, int page_rows, void* comp_pool, void* idx_pool,
                             float eps, int kv_row_bytes, int idx_row_bytes, void* stream) {
  if (idx_row_bytes != 0 && (idx_row_bytes < ID / 2 + ID / 32 || (ID & 31) || (idx_row_bytes & 3)))
    return cudaErrorInvalidValue;
  // kv_row_bytes: 0 bf16 rows, > 0 FP8 rows (D + D/32 bytes, padded), < 0 FP4 rows of -kv_row_bytes (D/2 + D/16 bytes)
  if (kv_row_bytes > 0 && (kv_row_bytes < D + D / 32 || (D & 31) || (kv_row_bytes & 15))) return cudaErrorInvalidValue;
  if (kv_row_bytes < 0 && (-kv_row_bytes < D / 2 + D / 16 || (D & 15) || ((-kv_row_bytes) & 15)))
    return cudaErrorInvalidValue;
  if (rows <= 0 || D > 1024 || ID > 256 || (ratio != 1 && ratio != 2) || (D & 1) || (ID & 3))
    return cudaErrorInvalidValue;
  CompressParams p{extras, extra_stride, rows, D, ID, rope_dim, ratio, row_pos, row_slot, pending, comp_norm_w,
                   static_cast<const __nv_bfloat16*>(wk), k_norm_w, inv_freq, inv_freq_idx, page_table, max_pages,
                   page_rows, static_cast<__nv_bfloat16*>(comp_pool), kv_row_bytes,
                   static_cast<__nv_bfloat16*>(idx_pool), eps, idx_row_bytes};
  return launch_pdl(compress_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}
