// Lightning-indexer scoring, exact top-k selection and sparse latent attention (decode / small-batch form).
//
//  index_score : score[r][c] = sum_h w[r][h] * relu(q[r][h] . key[c])   over the visible compressed rows
//                (native/cuda/kernels/v41_index_scores.cu:36-103)
//  topk_select : exact top-k by (score desc, row asc), emitted in ascending row order, all rows when
//                n_visible <= k (native/cuda/kernels/v41_index_topk.cu:25-124 semantics)
//  attend      : MQA over {window ring rows [pos-W+1, pos]} U {selected compressed rows}; K == V == one
//                latent of width D whose tail is rotary; per-head sink logit joins the softmax denominator;
//                keys are split across CTAs (64 per CTA) and merged, inverse RoPE applied to the output
//                (native/cuda/kernels/v41_sparse_attention.cu:89-381 semantics)
// The attention tiles use warp-level mma (m16n8k16 bf16): this kernel is latency/bandwidth bound at
// decode batch sizes, each CTA touching 64 gathered 1 KiB rows.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

__device__ __forceinline__ void rope_cs2(int pos, float inv_freq, float* c, float* s) {
  const double a = static_cast<double>(pos) * static_cast<double>(inv_freq);
  const double two_pi = 6.283185307179586476925286766559;
  const double red = a - floor(a * 0.15915494309189533576888376337251) * two_pi;
  sincosf(static_cast<float>(red), s, c);
}

__device__ __forceinline__ long long pool_row(const int* page_table, int max_pages, int page_rows, int slot, int id) {
  const int page = page_table[1ll * slot * max_pages + id / page_rows];
  return page < 0 ? -1ll : 1ll * page * page_rows + id % page_rows;
}

// ---------------------------------------------------------------------------------------- index score
struct IndexScoreParams {
  const __nv_bfloat16* q;     // [rows][ldq], index heads start at column q_off: [IH][ID]
  long long ldq;
  int q_off;
  const float* w;             // [rows][w_stride], head weights at column w_off
  int w_stride, w_off;
  const __nv_bfloat16* idx_pool;
  const int* page_table;
  int max_pages, page_rows;
  const int* row_pos;
  const int* row_slot;
  const float* inv_freq_idx;  // [ID/4]
  int rows, IH, ID, ratio;
  float* scores;              // [rows][max_keys]
  int max_keys;
  const uint32_t* cand_mask;  // optional [rows][cand_words]: one bit per block of cand_block keys; 0 = not scored
  int cand_words, cand_block;
  // > 0: key rows are FP4 (ID/2 bytes of E2M1 pairs, then ID/32 UE8M0 scales; idx_row_bytes apart) and the queries are
  // quantised to the same format before the dot; products are rounded to bf16 where the reference rounds them
  // (native/cuda/kernels/v41_index_scores.cu:36-103).  0: bf16 rows of ID values.
  int idx_row_bytes;
};

// two adjacent values of an FP4 key row
__device__ __forceinline__ float2 fp4_key_pair(const uint8_t* row, int ID, int d) {
  const uint32_t byte = row[d >> 1];
  const float scale = __uint_as_float(static_cast<uint32_t>(row[ID / 2 + (d >> 5)]) << 23);
  return make_float2(e2m1_value(byte & 15u) * scale, e2m1_value(byte >> 4) * scale);
}

__device__ __forceinline__ bool cand_allowed(const uint32_t* mask, int words, int block, int r, int key) {
  if (mask == nullptr) return true;
  const int b = key / block;
  return (mask[1ll * r * words + (b >> 5)] >> (b & 31)) & 1u;
}

// grid (blocks_x, rows), 256 threads; IH <= 32, ID <= 128
__global__ void __launch_bounds__(256) index_score_kernel(IndexScoreParams p) {
  __shared__ float qs[32][129];
  __shared__ float ws[32];
  __shared__ float kbuf[8][128];
  const int r = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.row_pos[r], slot = p.row_slot[r];
  if (slot < 0) return;
  const int n_vis = min((pos + 1) / p.ratio, p.max_keys);
  if (blockIdx.x * 8 >= n_vis) return;
  const int rope0 = p.ID - p.ID / 2;
  for (int idx = tid; idx < p.IH * p.ID / 2; idx += 256) {
    const unsigned lanes = __activemask();
    const int h = idx / (p.ID / 2), i = idx % (p.ID / 2);
    const float2 v = __bfloat1622float2(
        *reinterpret_cast<const __nv_bfloat162*>(p.q + 1ll * r * p.ldq + p.q_off + h * p.ID + 2 * i));
    float a = v.x, b = v.y;
    const int t = 2 * i - rope0;
    if (t >= 0) {
      float c, s;
      rope_cs2(pos, p.inv_freq_idx[t / 2], &c, &s);
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = bf16_round(ra);
      b = bf16_round(rb);
    }
    if (p.idx_row_bytes > 0) fp4_group_qdq(a, b, lanes);   // 16 consecutive threads hold one 32-value group of a head
    qs[h][2 * i] = a;
    qs[h][2 * i + 1] = b;
  }
  if (tid < 32) ws[tid] = tid < p.IH ? p.w[1ll * r * p.w_stride + p.w_off + tid] : 0.f;
  __syncthreads();
  for (int c = blockIdx.x * 8 + warp; c < n_vis; c += gridDim.x * 8) {
    if (!cand_allowed(p.cand_mask, p.cand_words, p.cand_block, r, c)) {      // warp-uniform: c is per warp
      if (lane == 0) p.scores[1ll * r * p.max_keys + c] = -INFINITY;
      continue;
    }
    const long long phys = pool_row(p.page_table, p.max_pages, p.page_rows, slot, c);
    __syncwarp();
    for (int d = lane * 2; d < p.ID; d += 64) {
      float2 v = make_float2(0.f, 0.f);
      if (phys >= 0)
        v = p.idx_row_bytes > 0
                ? fp4_key_pair(reinterpret_cast<const uint8_t*>(p.idx_pool) + phys * p.idx_row_bytes, p.ID, d)
                : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.idx_pool + phys * p.ID + d));
      kbuf[warp][d] = v.x;
      kbuf[warp][d + 1] = v.y;
    }
    __syncwarp();
    float acc = 0.f;
    if (lane < p.IH) {
      for (int d = 0; d < p.ID; ++d) acc = fmaf(qs[lane][d], kbuf[warp][d], acc);
      if (p.idx_row_bytes > 0) acc = bf16_round(fmaxf(bf16_round(acc), 0.f) * ws[lane]);   // the reference's rounding points
      else acc = fmaxf(acc, 0.f) * ws[lane];
    }
    acc = warp_sum(acc);
    if (p.idx_row_bytes > 0) acc = bf16_round(acc);
    if (lane == 0) p.scores[1ll * r * p.max_keys + c] = phys >= 0 ? acc : -INFINITY;
  }
}

// ---------------------------------------------------------------------------------------- index score on tensor cores
// Long passes over one request: the scores are a GEMM [rows*IH, ID] x [keys, ID]^T whose epilogue applies relu, the head
// weights and the sum over heads (gemm_tc.cu out_mode 8).  This kernel lays out its operands: blocks [0, rows) write the
// RoPE'd, bf16-rounded queries and the number of visible keys per row; the remaining blocks copy the request's index
// keys from the paged pool into one contiguous matrix (8 keys per block, zero rows where a page is missing).
__global__ void __launch_bounds__(256) index_prepare_kernel(IndexScoreParams p, int n_keys, __nv_bfloat16* qr,
                                                            __nv_bfloat16* kc, int* n_vis) {
  const int tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (static_cast<int>(blockIdx.x) < p.rows) {
    const int r = blockIdx.x;
    const int pos = p.row_pos[r], slot = p.row_slot[r];
    if (tid == 0) n_vis[r] = slot < 0 ? 0 : min(min((pos + 1) / p.ratio, p.max_keys), n_keys);
    const int rope0 = p.ID - p.ID / 2;
    for (int idx = tid; idx < p.IH * p.ID / 2; idx += 256) {
      const unsigned lanes = __activemask();
      const int h = idx / (p.ID / 2), i = idx % (p.ID / 2);
      const float2 v = __bfloat1622float2(
          *reinterpret_cast<const __nv_bfloat162*>(p.q + 1ll * r * p.ldq + p.q_off + h * p.ID + 2 * i));
      float a = v.x, b = v.y;
      const int t = 2 * i - rope0;
      if (t >= 0) {
        float c, s;
        rope_cs2(pos, p.inv_freq_idx[t / 2], &c, &s);
        const float ra = a * c - b * s, rb = b * c + a * s;
        a = ra;
        b = rb;
      }
      if (p.idx_row_bytes > 0) {
        a = bf16_round(a);
        b = bf16_round(b);
        fp4_group_qdq(a, b, lanes);
      }
      *reinterpret_cast<__nv_bfloat162*>(qr + (1ll * r * p.IH + h) * p.ID + 2 * i) = __floats2bfloat162_rn(a, b);
    }
    return;
  }
  const int slot = p.row_slot[0];
  const int vec = p.ID / 8;
  for (int idx = tid; idx < 8 * vec; idx += 256) {
    const int c = (blockIdx.x - p.rows) * 8 + idx / vec, v = idx % vec;
    if (c >= n_keys) continue;
    const long long phys = slot < 0 ? -1 : pool_row(p.page_table, p.max_pages, p.page_rows, slot, c);
    uint4 w = make_uint4(0, 0, 0, 0);
    if (phys >= 0 && p.idx_row_bytes > 0) {
      // FP4 key row -> eight bf16 values (every product of an E2M1 level and a power of two is a bf16 value)
      const uint8_t* row = reinterpret_cast<const uint8_t*>(p.idx_pool) + phys * p.idx_row_bytes;
      __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = fp4_key_pair(row, p.ID, v * 8 + 2 * j);
        o[j] = __floats2bfloat162_rn(f.x, f.y);
      }
    } else if (phys >= 0) {
      w = *reinterpret_cast<const uint4*>(p.idx_pool + phys * p.ID + v * 8);
    }
    *reinterpret_cast<uint4*>(kc + 1ll * c * p.ID + v * 8) = w;
  }
}

// ---------------------------------------------------------------------------------------- top-k
__device__ __forceinline__ uint32_t orderable(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One radix digit of the selection: given the 256-bin histogram of the keys that share the prefix found so far, find the
// highest bin d whose keys together with all keys in higher bins reach `need`, and how many keys of bin d are still
// needed.  Warp 0 does it: lane l sums bins 255 - 8l .. 248 - 8l, a shuffle scan gives the count above each lane's bins,
// and the one lane whose bins contain the answer walks its eight bins.  (One thread walking up to 255 bins, a dependent
// shared-memory load each, was most of the kernel's time: four digits per row.)
__device__ __forceinline__ void radix_pick(const int* hist, int need, uint32_t prefix, int shift, uint32_t* s_prefix,
                                           int* s_need) {
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  int local[8], sum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    local[j] = hist[255 - 8 * lane - j];
    sum += local[j];
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  const unsigned reach = __ballot_sync(0xffffffffu, incl >= need);
  const int owner = reach ? __ffs(reach) - 1 : 31;      // no lane reaches it: bin 0 takes what is left
  if (lane != owner) return;
  int cum = incl - sum, d = 255 - 8 * lane;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    d = 255 - 8 * lane - j;
    if (d == 0 || cum + local[j] >= need) break;
    cum += local[j];
  }
  *s_prefix = prefix | (static_cast<uint32_t>(d) << shift);
  *s_need = need - cum;
}

// exclusive scan over 1024 threads; returns this thread's exclusive prefix, *total gets the block sum
__device__ __forceinline__ int block_excl_scan_1024(int v, int* warp_tot /*[32]*/, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int t = warp_tot[lane];
    int ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += n;
    }
    warp_tot[lane] = ti - t;   // exclusive warp offsets
    if (lane == 31) *total = ti;
  }
  __syncthreads();
  return warp_tot[warp] + incl - v;
}

// Exact top-k of one row by a block of 1024 threads.  key(i) is the order-preserving 32-bit key of element i, 0 for an
// element that must never be chosen.  Writes the chosen ids in ascending order (-1 padded) and their count.  With at most
// k eligible elements all of them are chosen; otherwise a 4-pass radix select finds the k-th largest key and ties on it
// go to the lowest ids.
// Rows of at most 1024 * M elements: every thread keeps its M consecutive keys in registers, so the scores are read
// once, the four radix passes build their histograms from registers, and the ordered compaction needs two block scans
// in all (one block scan per 1024 elements and six reads of the row made the streaming form below take 30-43 us for 2 K
// to 16 K keys).
template <int M, class Key>
__device__ void select_topk_row_reg(Key key, int n, int k, int* out, int* n_out) {
  __shared__ int hist[256];
  __shared__ int warp_tot[32];
  __shared__ int s_total;
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  __shared__ int s_valid;
  const int tid = threadIdx.x;
  const int i0 = tid * M;
  uint32_t u[M];
  int mine = 0;
#pragma unroll
  for (int j = 0; j < M; ++j) {
    u[j] = i0 + j < n ? key(i0 + j) : 0u;
    mine += u[j] != 0u;
  }
  if (tid == 0) s_valid = 0;
  __syncthreads();
  if (mine) atomicAdd(&s_valid, mine);
  __syncthreads();
  const int valid = s_valid;
  for (int i = valid + tid; i < k; i += 1024) out[i] = -1;
  uint32_t thr = 0;
  int need = 0;
  if (valid > k) {
    uint32_t prefix = 0, mask = 0;
    need = k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < M; ++j)
        if (u[j] != 0u && (u[j] & mask) == prefix) atomicAdd(&hist[(u[j] >> shift) & 255], 1);
      __syncthreads();
      radix_pick(hist, need, prefix, shift, &s_prefix, &s_need);
      __syncthreads();
      prefix = s_prefix;
      need = s_need;
      mask |= 0xFFu << shift;
      __syncthreads();
    }
    thr = prefix;
  }
  // ordered compaction: ids ascend with the thread index, so one scan of the per-thread counts places every element
  int n_eq = 0;
#pragma unroll
  for (int j = 0; j < M; ++j) n_eq += (u[j] != 0u && u[j] == thr) ? 1 : 0;
  int eq_rank = block_excl_scan_1024(n_eq, warp_tot, &s_total);
  __syncthreads();
  int n_keep = 0;
  uint32_t keep_bits = 0;
#pragma unroll
  for (int j = 0; j < M; ++j) {
    const bool eq = u[j] != 0u && u[j] == thr;
    const bool keep = u[j] != 0u && (u[j] > thr || (eq && eq_rank < need));
    eq_rank += eq ? 1 : 0;
    keep_bits |= keep ? (1u << j) : 0u;
    n_keep += keep ? 1 : 0;
  }
  int at = block_excl_scan_1024(n_keep, warp_tot, &s_total);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < M; ++j)
    if ((keep_bits >> j) & 1u) {
      if (at < k) out[at] = i0 + j;
      ++at;
    }
  if (tid == 0) *n_out = min(s_total, k);
}

template <class Key>
__device__ void select_topk_row_stream(Key key, int n, int k, int* out, int* n_out) {
  __shared__ int hist[256];
  __shared__ int warp_tot[32];
  __shared__ int s_total;
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  __shared__ int s_valid;
  const int tid = threadIdx.x;
  if (tid == 0) s_valid = 0;
  __syncthreads();
  int mine = 0;
  for (int i = tid; i < n; i += 1024) mine += key(i) != 0u;
  if (mine) atomicAdd(&s_valid, mine);
  __syncthreads();
  const int valid = s_valid;
  for (int i = valid + tid; i < k; i += 1024) out[i] = -1;
  uint32_t thr = 0;
  int need = 0;
  if (valid > k) {
    uint32_t prefix = 0, mask = 0;
    need = k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int i = tid; i < n; i += 1024) {
        const uint32_t u = key(i);
        if (u != 0u && (u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1);
      }
      __syncthreads();
      radix_pick(hist, need, prefix, shift, &s_prefix, &s_need);
      __syncthreads();
      prefix = s_prefix;
      need = s_need;
      mask |= 0xFFu << shift;
      __syncthreads();
    }
    thr = prefix;                   // exact key of the k-th largest element; `need` of the equal ones are kept
  }
  // ---- ordered compaction (ascending id): keep key > thr, and the first `need` keys == thr
  int base = 0, eq_base = 0;
  for (int c0 = 0; c0 < n; c0 += 1024) {
    const int i = c0 + tid;
    uint32_t u = 0;
    if (i < n) u = key(i);
    const int is_eq = (i < n && u != 0u && u == thr) ? 1 : 0;
    int eq_total;
    const int eq_rank = eq_base + block_excl_scan_1024(is_eq, warp_tot, &s_total);
    __syncthreads();
    eq_total = s_total;
    const int keep = (i < n && u != 0u && (u > thr || (is_eq && eq_rank < need))) ? 1 : 0;
    const int at = base + block_excl_scan_1024(keep, warp_tot, &s_total);
    __syncthreads();
    if (keep && at < k) out[at] = i;
    base += s_total;
    eq_base += eq_total;
    __syncthreads();
  }
  if (tid == 0) *n_out = min(base, k);
}

template <class Key>
__device__ void select_topk_row(Key key, int n, int k, int* out, int* n_out) {
  if (n <= 4 * 1024) select_topk_row_reg<4>(key, n, k, out, n_out);
  else if (n <= 8 * 1024) select_topk_row_reg<8>(key, n, k, out, n_out);
  else if (n <= 16 * 1024) select_topk_row_reg<16>(key, n, k, out, n_out);
  else if (n <= 24 * 1024) select_topk_row_reg<24>(key, n, k, out, n_out);
  else select_topk_row_stream(key, n, k, out, n_out);
}

struct TopkParams {
  const float* scores;   // [rows][max_keys]
  int max_keys;
  const int* row_pos;
  const int* row_slot;
  int ratio, k;
  int* sel;              // [rows][k]  ascending ids, -1 padded
  int* n_sel;            // [rows]
  const uint32_t* cand_mask;   // optional [rows][cand_words]: keys of blocks whose bit is 0 are not eligible
  int cand_words, cand_block;
};

__global__ void __launch_bounds__(1024) topk_select_kernel(TopkParams p) {
  const int r = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.row_pos[r];
  int* out = p.sel + 1ll * r * p.k;
  if (p.row_slot[r] < 0) {
    for (int i = tid; i < p.k; i += 1024) out[i] = -1;
    if (tid == 0) p.n_sel[r] = 0;
    return;
  }
  const int n = min((pos + 1) / p.ratio, p.max_keys);
  if (n <= p.k && p.cand_mask == nullptr) {
    for (int i = tid; i < p.k; i += 1024) out[i] = i < n ? i : -1;
    if (tid == 0) p.n_sel[r] = n;
    return;
  }
  const float* sc = p.scores + 1ll * r * p.max_keys;
  const uint32_t* cm = p.cand_mask;
  const int words = p.cand_words, blk = p.cand_block;
  select_topk_row(
      [=](int i) -> uint32_t {
        if (!cand_allowed(cm, words, blk, r, i)) return 0u;
        const uint32_t u = orderable(sc[i]);
        return u == 0u ? 1u : u;
      },
      n, p.k, out, p.n_sel + r);
}

// Candidate blocks: the scores of one index layer are reduced to one score per block of `block` consecutive keys (the
// maximum), the newest visible block is pinned, the best `k_blocks` blocks are chosen and published both as a list
// (ascending block ids) and as a bit mask that the later index layers use to restrict scoring and selection.
struct CandParams {
  const float* scores;   // [rows][max_keys]
  int max_keys;
  const int* row_pos;
  const int* row_slot;
  int ratio, block, k_blocks;
  int* blocks;           // [rows][k_blocks]
  int* n_blocks;         // [rows]
  uint32_t* mask;        // [rows][words]
  int words;
};

__global__ void __launch_bounds__(1024) candidate_select_kernel(CandParams p) {
  const int r = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  uint32_t* mask = p.mask + 1ll * r * p.words;
  int* out = p.blocks + 1ll * r * p.k_blocks;
  for (int i = tid; i < p.words; i += 1024) mask[i] = 0u;
  const int n_vis = p.row_slot[r] < 0 ? 0 : min((p.row_pos[r] + 1) / p.ratio, p.max_keys);
  const int nb = (n_vis + p.block - 1) / p.block;
  if (nb == 0) {
    for (int i = tid; i < p.k_blocks; i += 1024) out[i] = -1;
    if (tid == 0) p.n_blocks[r] = 0;
    return;
  }
  const float* sc = p.scores + 1ll * r * p.max_keys;
  const int B = p.block, newest = (n_vis - 1) / B;
  select_topk_row(
      [=](int b) -> uint32_t {
        if (b == newest) return 0xFFFFFFFFu;
        float m = -INFINITY;
        const int hi = min(B, n_vis - b * B);
        for (int j = 0; j < hi; ++j) m = fmaxf(m, sc[b * B + j]);
        const uint32_t u = orderable(m);
        return u == 0u ? 1u : u;
      },
      nb, p.k_blocks, out, p.n_blocks + r);
  __syncthreads();                    // the list and its count (written by this block) are visible to all threads
  const int n = p.n_blocks[r];
  for (int i = tid; i < n; i += 1024) {
    const int b = out[i];
    atomicOr(&mask[b >> 5], 1u << (b & 31));
  }
}

// ---------------------------------------------------------------------------------------- attention
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(smem_u32(smem_row)));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                            const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(smem_u32(smem_row)));
}

struct AttendParams {
  const __nv_bfloat16* q;      // [rows][ldq]; local head h at column q_off + h*D
  long long ldq;
  int q_off;
  int rows, heads, window, ring;
  const int* row_pos;
  const int* row_slot;
  const __nv_bfloat16* win;    // [slots][ring][D]
  const __nv_bfloat16* comp_pool;   // may be null (window-only layer)
  const int* sel;              // [rows][k]
  const int* n_sel;            // [rows]
  int k;
  const int* page_table;
  int max_pages, page_rows;
  const float* inv_freq;       // [rope_dim/2]
  int rope_dim;
  float scale;
  int n_splits;
  const int* row_hi;           // optional [rows]: highest visible window position (>= pos); null = causal
  float* part_o;               // [rows][n_splits][heads][D]
  float* part_ml;              // [rows][n_splits][heads][2]
  int kv_row_bytes;            // 0: win / comp_pool rows are bf16 [D]; else FP8 rows (D e4m3 + D/32 UE8M0, padded)
  const int* row_lo;           // optional [rows]: lowest visible window position (a window rebuilt from there on)
  int comp_row_bytes;          // > 0: comp_pool rows are FP4 (D/2 e2m1 bytes + D/16 E4M3 scales) of this many bytes;
                               // the window rows must then be FP8 rows (kv_row_bytes > 0)
};

// Eight values of an FP4 cache row -> bf16 (exact: a 2-bit-mantissa value times a 4-bit-mantissa scale).
__device__ __forceinline__ uint4 expand_fp4_chunk(const uint8_t* row8, int D, int ch) {
  const uint32_t packed = *reinterpret_cast<const uint32_t*>(row8 + ch * 4);
  const __half_raw hs = __nv_cvt_fp8_to_halfraw(row8[D / 2 + (ch >> 1)], __NV_E4M3);
  const float sc = __half2float(__half(hs));
  uint4 out;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int q = 0; q < 4; ++q)
    o2[q] = __floats2bfloat162_rn(e2m1_value((packed >> (8 * q)) & 15u) * sc, e2m1_value((packed >> (8 * q + 4)) & 15u) * sc);
  return out;
}

constexpr int kKeysPerCta = 64;
constexpr int kHeadsPerCta = 16;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// grid (n_splits, rows, ceil(heads/16)), 128 threads: one CTA = 16 heads x the 64-key tiles split, split + n_splits, ...
// of one row, folded with a running softmax; n_splits = number of tiles gives one tile per CTA (decode), a small
// n_splits keeps the partial outputs of long passes small (prefill).
template <int D>
__global__ void __launch_bounds__(128) attend_kernel(AttendParams p) {
  constexpr int LD = D + 8;                                // padded row (bf16 elements)
  extern __shared__ __align__(16) uint8_t smem_attn[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_attn);                 // [64][LD]
  __nv_bfloat16* sQ = sK + kKeysPerCta * LD;                                         // [16][LD]
  float* sS = reinterpret_cast<float*>(sQ + kHeadsPerCta * LD);                      // [16][65]
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sS + kHeadsPerCta * 65);      // [16][72]
  float* sCos = reinterpret_cast<float*>(sP + kHeadsPerCta * 72);                    // [64]
  float* sSin = sCos + 64;
  const __nv_bfloat16** sPtr = reinterpret_cast<const __nv_bfloat16**>(sSin + 64);   // [64]
  float* sM = reinterpret_cast<float*>(sPtr + 64);                                    // [16] running max
  float* sL = sM + kHeadsPerCta;                                                      // [16] running sum
  float* sScale = sL + kHeadsPerCta;                                                  // [16] rescale of this tile
  uint8_t* sK8 = reinterpret_cast<uint8_t*>(sScale + kHeadsPerCta);                   // FP8 rows: [64][kv_row_bytes]

  const int split = blockIdx.x, r = blockIdx.y, h_base = blockIdx.z * kHeadsPerCta;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int n_heads = min(kHeadsPerCta, p.heads - h_base);
  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.row_pos[r], slot = p.row_slot[r];
  float* ml_out = p.part_ml + ((1ll * r * p.n_splits + split) * p.heads + h_base) * 2;
  float* o_out = p.part_o + ((1ll * r * p.n_splits + split) * p.heads + h_base) * D;

  int n_w = 0, n_s = 0, hi_pos = pos, lo_pos = 0;
  if (slot >= 0) {
    // drafter rows may see later rows of their own block: row_hi gives the highest visible position
    if (p.row_hi != nullptr) hi_pos = max(pos, p.row_hi[r]);
    lo_pos = max(0, pos - p.window + 1);
    if (p.row_lo != nullptr) lo_pos = max(lo_pos, p.row_lo[r]);
    n_w = hi_pos - lo_pos + 1;
    n_s = (p.comp_pool != nullptr && p.n_sel != nullptr) ? p.n_sel[r] : 0;
  }
  const int n_keys = n_w + n_s;
  const int n_tiles = (n_keys + kKeysPerCta - 1) / kKeysPerCta;
  if (split >= n_tiles) {
    if (tid < n_heads) {
      ml_out[2 * tid] = -INFINITY;
      ml_out[2 * tid + 1] = 0.f;
    }
    return;
  }
  // ---- rope table and the Q tile with RoPE on the tail (zero rows for padding heads), once per CTA
  if (tid < p.rope_dim / 2) rope_cs2(pos, p.inv_freq[tid], &sCos[tid], &sSin[tid]);
  if (tid < kHeadsPerCta) {
    sM[tid] = -INFINITY;
    sL[tid] = 0.f;
  }
  __syncthreads();
  const int rope0 = D - p.rope_dim;
#pragma unroll 4
  for (int idx = tid; idx < kHeadsPerCta * (D / 8); idx += 128) {
    const int h = idx / (D / 8), ch = idx % (D / 8);
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (h < n_heads)
      raw = *reinterpret_cast<const uint4*>(p.q + 1ll * r * p.ldq + p.q_off + 1ll * (h_base + h) * D + ch * 8);
    if (ch * 8 >= rope0 && h < n_heads) {
      __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(v[q]);
        const int t = (ch * 8 + 2 * q - rope0) / 2;
        const float c = sCos[t], sn = sSin[t];
        v[q] = __floats2bfloat162_rn(f.x * c - f.y * sn, f.y * c + f.x * sn);
      }
    }
    *reinterpret_cast<uint4*>(sQ + h * LD + ch * 8) = raw;
  }
  constexpr int NT = D / 32;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[nt][j] = 0.f;
  const int d_base = warp * (D / 4);

  // ---- this CTA's key tiles: split, split + n_splits, ... with a running (max, sum, output) per head
  for (int tile = split; tile < n_tiles; tile += p.n_splits) {
    const int k0 = tile * kKeysPerCta;
    const int k_cnt = min(kKeysPerCta, n_keys - k0);
    if (tid < kKeysPerCta) {
      const __nv_bfloat16* ptr = nullptr;
      const int j = k0 + tid;
      const long long row_bytes = p.kv_row_bytes > 0 ? p.kv_row_bytes : 2ll * D;
      if (tid < k_cnt) {
        if (j < n_w) {
          const int kp = lo_pos + j;
          ptr = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const uint8_t*>(p.win) +
                                                       (1ll * slot * p.ring + (kp % p.ring)) * row_bytes);
        } else {
          const int id = p.sel[1ll * r * p.k + (j - n_w)];
          const long long phys = id < 0 ? -1 : pool_row(p.page_table, p.max_pages, p.page_rows, slot, id);
          if (phys >= 0)
            ptr = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const uint8_t*>(p.comp_pool) +
                                                         phys * (p.comp_row_bytes > 0 ? p.comp_row_bytes : row_bytes));
        }
      }
      sPtr[tid] = ptr;
    }
    __syncthreads();          // also: the previous tile's P.V reads of sK / sP are complete
    // K tile: asynchronous 16-byte copies straight into shared memory (zero-filled beyond k_cnt)
    if (p.kv_row_bytes == 0) {
#pragma unroll 8
      for (int idx = tid; idx < kKeysPerCta * (D / 8); idx += 128) {
        const int key = idx / (D / 8), ch = idx % (D / 8);
        const __nv_bfloat16* src = sPtr[key];
        __nv_bfloat16* dst = sK + key * LD + ch * 8;
        if (src != nullptr) cp_async_16(dst, src + ch * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
      cp_async_wait_all();
      __syncthreads();
    } else {
      // FP8 rows: copy payload + scales as they are, then expand to bf16 (exact: e4m3 value times a power of two)
      const int chunks = p.kv_row_bytes / 16;
      const int comp_chunks = p.comp_row_bytes > 0 ? p.comp_row_bytes / 16 : chunks;
      for (int idx = tid; idx < kKeysPerCta * chunks; idx += 128) {
        const int key = idx / chunks, ch = idx - key * chunks;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(sPtr[key]);
        uint8_t* dst = sK8 + key * p.kv_row_bytes + ch * 16;
        if (src == nullptr) *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        else if (ch < (k0 + key >= n_w ? comp_chunks : chunks)) cp_async_16(dst, src + ch * 16);   // FP4 rows are shorter
      }
      cp_async_wait_all();
      __syncthreads();
#pragma unroll 4
      for (int idx = tid; idx < kKeysPerCta * (D / 8); idx += 128) {
        const int key = idx / (D / 8), ch = idx % (D / 8);
        const uint8_t* row8 = sK8 + key * p.kv_row_bytes;
        if (p.comp_row_bytes > 0 && k0 + key >= n_w) {
          *reinterpret_cast<uint4*>(sK + key * LD + ch * 8) = expand_fp4_chunk(row8, D, ch);
          continue;
        }
        const uint2 raw = *reinterpret_cast<const uint2*>(row8 + ch * 8);
        const float sc = __uint_as_float(static_cast<uint32_t>(row8[D + (ch >> 2)]) << 23);
        const __nv_fp8x2_storage_t* q2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
        uint4 out;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(q2[q], __NV_E4M3)));
          o2[q] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
        *reinterpret_cast<uint4*>(sK + key * LD + ch * 8) = out;
      }
      __syncthreads();
    }
    // S = Q K^T: warp w owns keys [16w, 16w+16)
    {
      float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const __nv_bfloat16* qa = sQ + g * LD + 2 * t4;
      const __nv_bfloat16* kb = sK + (warp * 16 + g) * LD + 2 * t4;
#pragma unroll 8
      for (int kk = 0; kk < D; kk += 16) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(qa + kk);
        a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * LD + kk);
        a[2] = *reinterpret_cast<const uint32_t*>(qa + kk + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * LD + kk + 8);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kb + nt * 8 * LD + kk);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kb + nt * 8 * LD + kk + 8);
          mma_bf16_16816(c[nt], a, b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int key = warp * 16 + nt * 8 + 2 * t4;
        float* s0 = sS + g * 65 + key;
        float* s1 = sS + (g + 8) * 65 + key;
        s0[0] = key < k_cnt ? c[nt][0] * p.scale : -INFINITY;
        s0[1] = key + 1 < k_cnt ? c[nt][1] * p.scale : -INFINITY;
        s1[0] = key < k_cnt ? c[nt][2] * p.scale : -INFINITY;
        s1[1] = key + 1 < k_cnt ? c[nt][3] * p.scale : -INFINITY;
      }
    }
    __syncthreads();
    // per-head running softmax statistics; P in bf16 (4 head rows per warp)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = warp * 4 + i;
      const float v0 = sS[row * 65 + lane], v1 = sS[row * 65 + lane + 32];
      const float m_old = sM[row];
      const float m = fmaxf(m_old, warp_max(fmaxf(v0, v1)));
      const float e0 = __expf(v0 - m), e1 = __expf(v1 - m);
      const __nv_bfloat16 b0 = __float2bfloat16_rn(e0), b1 = __float2bfloat16_rn(e1);
      const float l = warp_sum(__bfloat162float(b0) + __bfloat162float(b1));
      sP[row * 72 + lane] = b0;
      sP[row * 72 + lane + 32] = b1;
      if (lane == 0) {
        const float keep = m_old == -INFINITY ? 0.f : __expf(m_old - m);
        sScale[row] = keep;
        sL[row] = sL[row] * keep + l;
        sM[row] = m;
      }
    }
    __syncthreads();
    // O = O * keep + P V : warp w owns dims [w*D/4, (w+1)*D/4)
    {
      const float keep0 = sScale[g], keep1 = sScale[g + 8];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        acc[nt][0] *= keep0;
        acc[nt][1] *= keep0;
        acc[nt][2] *= keep1;
        acc[nt][3] *= keep1;
      }
#pragma unroll
      for (int kk = 0; kk < kKeysPerCta; kk += 16) {
        uint32_t a[4];
        const __nv_bfloat16* pa = sP + g * 72 + kk + 2 * t4;
        a[0] = *reinterpret_cast<const uint32_t*>(pa);
        a[1] = *reinterpret_cast<const uint32_t*>(pa + 8 * 72);
        a[2] = *reinterpret_cast<const uint32_t*>(pa + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(pa + 8 * 72 + 8);
        const __nv_bfloat16* vrow = sK + (kk + (lane & 15)) * LD + d_base;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t b0, b1;
          ldmatrix_x2_trans(b0, b1, vrow + nt * 8);
          mma_bf16_16816(acc[nt], a, b0, b1);
        }
      }
    }
  }
  __syncthreads();
  if (tid < n_heads) {
    ml_out[2 * tid] = sM[tid];
    ml_out[2 * tid + 1] = sL[tid];
  }
  {
    const int h0 = g, h1 = g + 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int d = d_base + nt * 8 + 2 * t4;
      if (h0 < n_heads) *reinterpret_cast<float2*>(o_out + 1ll * h0 * D + d) = make_float2(acc[nt][0], acc[nt][1]);
      if (h1 < n_heads) *reinterpret_cast<float2*>(o_out + 1ll * h1 * D + d) = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
}

// ---------------------------------------------------------------------------------------- wide variant (long passes)
// grid (n_splits, rows, heads/64), 512 threads: one CTA = all 64 heads of a head block x this split's keys of one row.
// The gathered latent rows are shared by the four 16-head groups (a quarter of the gather traffic of attend_kernel), in
// half tiles of 32 keys that are double buffered: the copies of half tile i+1 are in flight while half tile i is used.
// Warp w: head group w & 3, part w >> 2.  S = Q K^T: 16 heads x 8 keys per warp; softmax: 4 heads per warp (lane =
// key); O += P V: 16 heads x D/4 dims per warp.  Split partials and the merge kernel are the same as attend_kernel's.
constexpr int kWideHeads = 64;
constexpr int kWideKeys = 32;

template <int D>
__global__ void __launch_bounds__(512) attend_wide_kernel(AttendParams p) {
  constexpr int LD = D + 8;
  extern __shared__ __align__(16) uint8_t smem_attn[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_attn);                    // [64][LD]
  __nv_bfloat16* sK = sQ + kWideHeads * LD;                                           // [2][32][LD]
  float* sS = reinterpret_cast<float*>(sK + 2 * kWideKeys * LD);                      // [64][33]
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sS + kWideHeads * 33);         // [64][40]
  float* sCos = reinterpret_cast<float*>(sP + kWideHeads * 40);                       // [64]
  float* sSin = sCos + 64;
  const __nv_bfloat16** sPtr = reinterpret_cast<const __nv_bfloat16**>(sSin + 64);    // [2][32]
  float* sM = reinterpret_cast<float*>(sPtr + 2 * kWideKeys);                         // [64]
  float* sL = sM + kWideHeads;
  float* sScale = sL + kWideHeads;
  uint8_t* sK8 = reinterpret_cast<uint8_t*>(sScale + kWideHeads);                     // FP8 rows: [2][32][kv_row_bytes]

  const int split = blockIdx.x, r = blockIdx.y, h_base = blockIdx.z * kWideHeads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int hg = warp & 3, part = warp >> 2;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.row_pos[r], slot = p.row_slot[r];
  float* ml_out = p.part_ml + ((1ll * r * p.n_splits + split) * p.heads + h_base) * 2;
  float* o_out = p.part_o + ((1ll * r * p.n_splits + split) * p.heads + h_base) * D;

  int n_w = 0, n_s = 0, hi_pos = pos, lo_pos = 0;
  if (slot >= 0) {
    if (p.row_hi != nullptr) hi_pos = max(pos, p.row_hi[r]);
    lo_pos = max(0, pos - p.window + 1);
    if (p.row_lo != nullptr) lo_pos = max(lo_pos, p.row_lo[r]);
    n_w = hi_pos - lo_pos + 1;
    n_s = (p.comp_pool != nullptr && p.n_sel != nullptr) ? p.n_sel[r] : 0;
  }
  const int n_keys = n_w + n_s;
  const int n_half = (n_keys + kWideKeys - 1) / kWideKeys;      // half tiles of this row
  // split s takes half tiles s, s + n_splits, ...
  if (split >= n_half) {
    if (tid < kWideHeads) {
      ml_out[2 * tid] = -INFINITY;
      ml_out[2 * tid + 1] = 0.f;
    }
    return;
  }
  if (tid < p.rope_dim / 2) rope_cs2(pos, p.inv_freq[tid], &sCos[tid], &sSin[tid]);
  if (tid < kWideHeads) {
    sM[tid] = -INFINITY;
    sL[tid] = 0.f;
  }
  const long long row_bytes = p.kv_row_bytes > 0 ? p.kv_row_bytes : 2ll * D;

  // pointer table + copies of one half tile into buffer b (every thread commits one group per call)
  auto issue = [&](int half, int b) {
    const int k0 = half * kWideKeys;
    const int k_cnt = min(kWideKeys, n_keys - k0);
    if (tid < kWideKeys) {
      const __nv_bfloat16* ptr = nullptr;
      const int j = k0 + tid;
      if (tid < k_cnt) {
        if (j < n_w) {
          const int kp = lo_pos + j;
          ptr = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const uint8_t*>(p.win) +
                                                       (1ll * slot * p.ring + (kp % p.ring)) * row_bytes);
        } else {
          const int id = p.sel[1ll * r * p.k + (j - n_w)];
          const long long phys = id < 0 ? -1 : pool_row(p.page_table, p.max_pages, p.page_rows, slot, id);
          if (phys >= 0)
            ptr = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const uint8_t*>(p.comp_pool) +
                                                         phys * (p.comp_row_bytes > 0 ? p.comp_row_bytes : row_bytes));
        }
      }
      sPtr[b * kWideKeys + tid] = ptr;
    }
    __syncthreads();
    if (p.kv_row_bytes == 0) {
      for (int idx = tid; idx < kWideKeys * (D / 8); idx += 512) {
        const int key = idx / (D / 8), ch = idx % (D / 8);
        const __nv_bfloat16* src = sPtr[b * kWideKeys + key];
        __nv_bfloat16* dst = sK + (b * kWideKeys + key) * LD + ch * 8;
        if (src != nullptr) cp_async_16(dst, src + ch * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    } else {
      const int chunks = p.kv_row_bytes / 16;
      const int comp_chunks = p.comp_row_bytes > 0 ? p.comp_row_bytes / 16 : chunks;
      for (int idx = tid; idx < kWideKeys * chunks; idx += 512) {
        const int key = idx / chunks, ch = idx - key * chunks;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(sPtr[b * kWideKeys + key]);
        uint8_t* dst = sK8 + (b * kWideKeys + key) * p.kv_row_bytes + ch * 16;
        if (src == nullptr) *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        else if (ch < (k0 + key >= n_w ? comp_chunks : chunks)) cp_async_16(dst, src + ch * 16);   // FP4 rows are shorter
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  issue(split, 0);
  // Q tile with RoPE on the tail (zero rows for heads beyond this rank's count), while the first copies fly
  const int rope0 = D - p.rope_dim;
  const int n_heads = min(kWideHeads, p.heads - h_base);
  for (int idx = tid; idx < kWideHeads * (D / 8); idx += 512) {
    const int h = idx / (D / 8), ch = idx % (D / 8);
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (h < n_heads)
      raw = *reinterpret_cast<const uint4*>(p.q + 1ll * r * p.ldq + p.q_off + 1ll * (h_base + h) * D + ch * 8);
    if (ch * 8 >= rope0 && h < n_heads) {
      __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(v[q]);
        const int t = (ch * 8 + 2 * q - rope0) / 2;
        const float c = sCos[t], sn = sSin[t];
        v[q] = __floats2bfloat162_rn(f.x * c - f.y * sn, f.y * c + f.x * sn);
      }
    }
    *reinterpret_cast<uint4*>(sQ + h * LD + ch * 8) = raw;
  }
  constexpr int NT = D / 32;                 // n8 tiles of this warp's D/4 output dims
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[nt][j] = 0.f;
  const int d_base = part * (D / 4);

  int buf = 0;
  for (int half = split; half < n_half; half += p.n_splits, buf ^= 1) {
    const int k0 = half * kWideKeys;
    const int k_cnt = min(kWideKeys, n_keys - k0);
    const int next = half + p.n_splits;
    if (next < n_half) {
      issue(next, buf ^ 1);                  // its buffer was last read two iterations ago (sync at the loop's end)
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    __nv_bfloat16* kt = sK + buf * kWideKeys * LD;
    if (p.kv_row_bytes != 0) {
      // FP8 rows -> bf16 (exact: e4m3 value times a power of two)
      for (int idx = tid; idx < kWideKeys * (D / 8); idx += 512) {
        const int key = idx / (D / 8), ch = idx % (D / 8);
        const uint8_t* row8 = sK8 + (buf * kWideKeys + key) * p.kv_row_bytes;
        if (p.comp_row_bytes > 0 && k0 + key >= n_w) {
          *reinterpret_cast<uint4*>(kt + key * LD + ch * 8) = expand_fp4_chunk(row8, D, ch);
          continue;
        }
        const uint2 raw = *reinterpret_cast<const uint2*>(row8 + ch * 8);
        const float sc = __uint_as_float(static_cast<uint32_t>(row8[D + (ch >> 2)]) << 23);
        const __nv_fp8x2_storage_t* q2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
        uint4 out;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(q2[q], __NV_E4M3)));
          o2[q] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
        *reinterpret_cast<uint4*>(kt + key * LD + ch * 8) = out;
      }
      __syncthreads();
    }
    // ---- S = Q K^T: this warp's 16 heads x 8 keys
    {
      // fragments come from ldmatrix: one x4 per 16 x 16 block of Q and one x4 per two k-steps of the 8 key rows
      // (three shared-memory instructions per two MMAs instead of twelve 32-bit loads)
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* qa = sQ + (hg * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
      const __nv_bfloat16* kb = kt + (part * 8 + (lane & 7)) * LD + (lane >> 3) * 8;
#pragma unroll 4
      for (int kk = 0; kk < D; kk += 32) {
        uint32_t a[4], a2[4], b[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], qa + kk);
        ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], qa + kk + 16);
        ldmatrix_x4(b[0], b[1], b[2], b[3], kb + kk);
        mma_bf16_16816(c, a, b[0], b[1]);
        mma_bf16_16816(c, a2, b[2], b[3]);
      }
      const int key = part * 8 + 2 * t4;
      float* s0 = sS + (hg * 16 + g) * 33 + key;
      float* s1 = sS + (hg * 16 + g + 8) * 33 + key;
      s0[0] = key < k_cnt ? c[0] * p.scale : -INFINITY;
      s0[1] = key + 1 < k_cnt ? c[1] * p.scale : -INFINITY;
      s1[0] = key < k_cnt ? c[2] * p.scale : -INFINITY;
      s1[1] = key + 1 < k_cnt ? c[3] * p.scale : -INFINITY;
    }
    __syncthreads();
    // ---- running softmax statistics, 4 heads per warp, lane = key
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = warp * 4 + i;
      const float v0 = sS[row * 33 + lane];
      const float m_old = sM[row];
      const float m = fmaxf(m_old, warp_max(v0));
      const float e0 = __expf(v0 - m);
      const __nv_bfloat16 b0 = __float2bfloat16_rn(e0);
      const float l = warp_sum(__bfloat162float(b0));
      sP[row * 40 + lane] = b0;
      if (lane == 0) {
        const float keep = m_old == -INFINITY ? 0.f : __expf(m_old - m);
        sScale[row] = keep;
        sL[row] = sL[row] * keep + l;
        sM[row] = m;
      }
    }
    __syncthreads();
    // ---- O = O * keep + P V: this warp's 16 heads x D/4 dims
    {
      const float keep0 = sScale[hg * 16 + g], keep1 = sScale[hg * 16 + g + 8];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        acc[nt][0] *= keep0;
        acc[nt][1] *= keep0;
        acc[nt][2] *= keep1;
        acc[nt][3] *= keep1;
      }
#pragma unroll
      for (int kk = 0; kk < kWideKeys; kk += 16) {
        uint32_t a[4];
        const __nv_bfloat16* pa = sP + (hg * 16 + g) * 40 + kk + 2 * t4;
        a[0] = *reinterpret_cast<const uint32_t*>(pa);
        a[1] = *reinterpret_cast<const uint32_t*>(pa + 8 * 40);
        a[2] = *reinterpret_cast<const uint32_t*>(pa + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(pa + 8 * 40 + 8);
        const __nv_bfloat16* vrow = kt + (kk + (lane & 15)) * LD + d_base + (lane >> 4) * 8;
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, vrow + nt * 8);      // two 8-column tiles of V per instruction
          mma_bf16_16816(acc[nt], a, b0, b1);
          mma_bf16_16816(acc[nt + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();     // everyone is done with this buffer, sS and sP
  }
  if (tid < n_heads) {
    ml_out[2 * tid] = sM[tid];
    ml_out[2 * tid + 1] = sL[tid];
  }
  {
    const int h0 = hg * 16 + g, h1 = h0 + 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int d = d_base + nt * 8 + 2 * t4;
      if (h0 < n_heads) *reinterpret_cast<float2*>(o_out + 1ll * h0 * D + d) = make_float2(acc[nt][0], acc[nt][1]);
      if (h1 < n_heads) *reinterpret_cast<float2*>(o_out + 1ll * h1 * D + d) = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
}

struct MergeParams {
  const float* part_o;
  const float* part_ml;
  const float* sink;        // [heads] (this rank's heads)
  const int* row_pos;
  const int* row_slot;
  const float* inv_freq;
  int rope_dim, heads, D, n_splits;
  __nv_bfloat16* out;       // [rows][ldo], head h at column h*D
  long long ldo;
};

// grid (heads, rows), 128 threads; n_splits <= 32
__global__ void __launch_bounds__(128) attend_merge_kernel(MergeParams p) {
  __shared__ float s_w[32];
  __shared__ float s_denom;
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (tid < 32) {
    // one warp: all splits' (m, l) at once, then the combined max and denominator
    const float sink = p.sink[h];
    float m_s = -INFINITY, l_s = 0.f;
    if (tid < p.n_splits) {
      const float* ml = p.part_ml + ((1ll * r * p.n_splits + tid) * p.heads + h) * 2;
      m_s = ml[0];
      l_s = ml[1];
    }
    const float m = fmaxf(warp_max(l_s > 0.f ? m_s : -INFINITY), sink);
    const float w = l_s > 0.f ? __expf(m_s - m) : 0.f;
    const float denom = warp_sum(w * l_s) + __expf(sink - m);
    s_w[tid] = w;
    if (tid == 0) s_denom = denom;
  }
  __syncthreads();
  const float inv_denom = 1.0f / s_denom;
  const int pos = p.row_pos[r];
  const int rope0 = p.D - p.rope_dim;
  const bool live = p.row_slot[r] >= 0;
  for (int i = tid; i < p.D / 2; i += 128) {
    float a = 0.f, b = 0.f;
    for (int s = 0; s < p.n_splits; ++s) {
      const float w = s_w[s];
      if (w > 0.f) {
        const float2 v = *reinterpret_cast<const float2*>(p.part_o + ((1ll * r * p.n_splits + s) * p.heads + h) * p.D + 2 * i);
        a = fmaf(w, v.x, a);
        b = fmaf(w, v.y, b);
      }
    }
    a *= inv_denom;
    b *= inv_denom;
    const int t = 2 * i - rope0;
    if (t >= 0) {
      float c, s;
      rope_cs2(pos, p.inv_freq[t / 2], &c, &s);
      const float ra = a * c + b * s, rb = b * c - a * s;     // inverse rotation
      a = ra;
      b = rb;
    }
    if (!live) { a = 0.f; b = 0.f; }
    *reinterpret_cast<__nv_bfloat162*>(p.out + 1ll * r * p.ldo + 1ll * h * p.D + 2 * i) = __floats2bfloat162_rn(a, b);
  }
}

template <int D>
static cudaError_t launch_attend(const AttendParams& p, cudaStream_t stream) {
  constexpr int LD = D + 8;
  constexpr size_t base = size_t(kKeysPerCta) * LD * 2 + size_t(kHeadsPerCta) * LD * 2 + size_t(kHeadsPerCta) * 65 * 4 +
                          size_t(kHeadsPerCta) * 72 * 2 + 128 * 4 + 64 * 8 + 3 * kHeadsPerCta * 4 + 64;
  constexpr size_t smem_max = base + size_t(kKeysPerCta) * ((D + D / 32 + 15) / 16 * 16);
  const size_t smem = base + size_t(kKeysPerCta) * p.kv_row_bytes;
  if (p.kv_row_bytes != 0 && (p.kv_row_bytes < D + D / 32 || (p.kv_row_bytes & 15) || smem > smem_max))
    return cudaErrorInvalidValue;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attend_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_max));
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  if (p.rows >= 64 && p.heads % kWideHeads == 0 && D % 128 == 0) {
    // long pass: all 64 heads of a block share every gathered key row
    const size_t wide = size_t(kWideHeads) * LD * 2 + 2 * size_t(kWideKeys) * LD * 2 + size_t(kWideHeads) * 33 * 4 +
                        size_t(kWideHeads) * 40 * 2 + 128 * 4 + 2 * kWideKeys * 8 + 3 * kWideHeads * 4 + 64 +
                        2 * size_t(kWideKeys) * p.kv_row_bytes;
    static bool wide_configured[64] = {false};
    if (dev >= 0 && dev < 64 && !wide_configured[dev]) {
      const size_t wide_max = wide - 2 * size_t(kWideKeys) * p.kv_row_bytes +
                              2 * size_t(kWideKeys) * ((D + D / 32 + 15) / 16 * 16);
      cudaError_t e = cudaFuncSetAttribute(attend_wide_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           int(wide_max));
      if (e != cudaSuccess) return e;
      wide_configured[dev] = true;
    }
    dim3 wgrid(p.n_splits, p.rows, p.heads / kWideHeads);
    return launch_pdl(attend_wide_kernel<D>, wgrid, dim3(512), wide, stream, p);
  }
  dim3 grid(p.n_splits, p.rows, (p.heads + kHeadsPerCta - 1) / kHeadsPerCta);
  return launch_pdl(attend_kernel<D>, grid, dim3(128), smem, stream, p);
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_index_score_cand(const void* q, long long ldq, int q_off, const float* w, int w_stride, int w_off,
                                     const void* idx_pool, const int* page_table, int max_pages, int page_rows,
                                     const int* row_pos, const int* row_slot, const float* inv_freq_idx, int rows,
                                     int IH, int ID, int ratio, float* scores, int max_keys, const void* cand_mask,
                                     int cand_words, int cand_block, int idx_row_bytes, void* stream) {
  if (rows <= 0 || IH > 32 || ID > 128 || (ID & 3)) return cudaErrorInvalidValue;
  if (idx_row_bytes != 0 && (idx_row_bytes < ID / 2 + ID / 32 || (ID & 31))) return cudaErrorInvalidValue;
  if (cand_mask != nullptr && (cand_words <= 0 || cand_block <= 0)) return cudaErrorInvalidValue;
  IndexScoreParams p{static_cast<const __nv_bfloat16*>(q), ldq, q_off, w, w_stride, w_off,
                     static_cast<const __nv_bfloat16*>(idx_pool), page_table, max_pages, page_rows, row_pos,
                     row_slot, inv_freq_idx, rows, IH, ID, ratio, scores, max_keys,
                     static_cast<const uint32_t*>(cand_mask), cand_words, cand_block, idx_row_bytes};
  int bx = (max_keys + 7) / 8;
  if (bx > 256) bx = 256;
  return launch_pdl(index_score_kernel, dim3(bx, rows), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_index_score(const void* q, long long ldq, int q_off, const float* w, int w_stride, int w_off,
                                const void* idx_pool, const int* page_table, int max_pages, int page_rows,
                                const int* row_pos, const int* row_slot, const float* inv_freq_idx, int rows, int IH,
                                int ID, int ratio, float* scores, int max_keys, void* stream) {
  return ds41_index_score_cand(q, ldq, q_off, w, w_stride, w_off, idx_pool, page_table, max_pages, page_rows, row_pos,
                               row_slot, inv_freq_idx, rows, IH, ID, ratio, scores, max_keys, nullptr, 0, 0, 0, stream);
}

extern "C" int ds41_index_prepare(const void* q, long long ldq, int q_off, const void* idx_pool, const int* page_table,
                                  int max_pages, int page_rows, const int* row_pos, const int* row_slot,
                                  const float* inv_freq_idx, int rows, int IH, int ID, int ratio, int n_keys,
                                  int max_keys, void* qr, void* kc, int* n_vis, int idx_row_bytes, void* stream) {
  if (rows <= 0 || n_keys <= 0 || IH <= 0 || ID <= 0 || (ID & 7)) return cudaErrorInvalidValue;
  if (idx_row_bytes != 0 && (idx_row_bytes < ID / 2 + ID / 32 || (ID & 31))) return cudaErrorInvalidValue;
  IndexScoreParams p{static_cast<const __nv_bfloat16*>(q), ldq, q_off, nullptr, 0, 0,
                     static_cast<const __nv_bfloat16*>(idx_pool), page_table, max_pages, page_rows, row_pos,
                     row_slot, inv_freq_idx, rows, IH, ID, ratio, nullptr, max_keys, nullptr, 0, 0, idx_row_bytes};
  return launch_pdl(index_prepare_kernel, dim3(rows + (n_keys + 7) / 8), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), p, n_keys, static_cast<__nv_bfloat16*>(qr),
                    static_cast<__nv_bfloat16*>(kc), n_vis);
}

extern "C" int ds41_topk_select_cand(const float* scores, int max_keys, const int* row_pos, const int* row_slot,
                                     int ratio, int k, int* sel, int* n_sel, int rows, const void* cand_mask,
                                     int cand_words, int cand_block, void* stream) {
  if (rows <= 0 || k <= 0) return cudaErrorInvalidValue;
  if (cand_mask != nullptr && (cand_words <= 0 || cand_block <= 0)) return cudaErrorInvalidValue;
  TopkParams p{scores, max_keys, row_pos, row_slot, ratio, k, sel, n_sel,
               static_cast<const uint32_t*>(cand_mask), cand_words, cand_block};
  return launch_pdl(topk_select_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_topk_select(const float* scores, int max_keys, const int* row_pos, const int* row_slot,
                                int ratio, int k, int* sel, int* n_sel, int rows, void* stream) {
  return ds41_topk_select_cand(scores, max_keys, row_pos, row_slot, ratio, k, sel, n_sel, rows, nullptr, 0, 0, stream);
}

extern "C" int ds41_candidate_select(const float* scores, int max_keys, const int* row_pos, const int* row_slot,
                                     int ratio, int block, int k_blocks, int* blocks, int* n_blocks, void* mask,
                                     int words, int rows, void* stream) {
  if (rows <= 0 || block <= 0 || k_blocks <= 0 || ratio <= 0 || scores == nullptr || blocks == nullptr ||
      n_blocks == nullptr || mask == nullptr || 32ll * words * block < max_keys)
    return cudaErrorInvalidValue;
  CandParams p{scores, max_keys, row_pos, row_slot, ratio, block, k_blocks, blocks, n_blocks,
               static_cast<uint32_t*>(mask), words};
  return launch_pdl(candidate_select_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_attend_merge(const float* part_o, const float* part_ml, const float* sink, const int* row_pos,
                                 const int* row_slot, const float* inv_freq, int rope_dim, int heads, int D, int n_splits,
                                 int rows, void* out, long long ldo, void* stream) {
  if (rows <= 0 || heads <= 0 || n_splits <= 0 || n_splits > 32 || (D & 1)) return cudaErrorInvalidValue;
  MergeParams m{part_o, part_ml, sink, row_pos, row_slot, inv_freq, rope_dim, heads, D, n_splits,
                static_cast<__nv_bfloat16*>(out), ldo};
  return launch_pdl(attend_merge_kernel, dim3(heads, rows), dim3(128), 0, static_cast<cudaStream_t>(stream), m);
}

extern "C" int ds41_attend(const void* q, long long ldq, int q_off, int rows, int heads, int D, int window, int ring,
                           const int* row_pos, const int* row_slot, const void* win, const void* comp_pool,
                           const int* sel, const int* n_sel, int k, const int* page_table, int max_pages,
                           int page_rows, const float* inv_freq, int rope_dim, float scale, int n_splits,
                           const int* row_hi, float* part_o, float* part_ml, const float* sink, void* out,
                           long long ldo, int kv_row_bytes, void* stream) {
  return ds41_attend_floor(q, ldq, q_off, rows, heads, D, window, ring, row_pos, row_slot, win, comp_pool, sel, n_sel, k,
                           page_table, max_pages, page_rows, inv_freq, rope_dim, scale, n_splits, row_hi, part_o,
                           part_ml, sink, out, ldo, kv_row_bytes, nullptr, stream);
}

extern "C" int ds41_attend_floor(const void* q, long long ldq, int q_off, int rows, int heads, int D, int window,
                                 int ring, const int* row_pos, const int* row_slot, const void* win,
                                 const void* comp_pool, const int* sel, const int* n_sel, int k, const int* page_table,
                                 int max_pages, int page_rows, const float* inv_freq, int rope_dim, float scale,
                                 int n_splits, const int* row_hi, float* part_o, float* part_ml, const float* sink,
                                 void* out, long long ldo, int kv_row_bytes, const int* row_lo, void* stream) {
  return ds41_attend_kv(q, ldq, q_off, rows, heads, D, window, ring, row_pos, row_slot, win, comp_pool, sel, n_sel, k,
                        page_table, max_pages, page_rows, inv_freq, rope_dim, scale, n_splits, row_hi, part_o, part_ml,
                        sink, out, ldo, kv_row_bytes, 0, row_lo, stream);
}

extern "C" int ds41_attend_kv(const void* q, long long ldq, int q_off, int rows, int heads, int D, int window,
                              int ring, const int* row_pos, const int* row_slot, const void* win,
                              const void* comp_pool, const int* sel, const int* n_sel, int k, const int* page_table,
                              int max_pages, int page_rows, const float* inv_freq, int rope_dim, float scale,
                              int n_splits, const int* row_hi, float* part_o, float* part_ml, const float* sink,
                              void* out, long long ldo, int kv_row_bytes, int comp_row_bytes, const int* row_lo,
                              void* stream) {
  if (comp_row_bytes != 0 && (kv_row_bytes <= 0 || comp_row_bytes < D / 2 + D / 16 || (comp_row_bytes & 15) ||
                              comp_row_bytes > kv_row_bytes))
    return cudaErrorInvalidValue;
  if (rows <= 0 || heads <= 0 || rope_dim > 128 || (rope_dim & 7) || n_splits <= 0 || n_splits > 32)
    return cudaErrorInvalidValue;
  AttendParams p{static_cast<const __nv_bfloat16*>(q), ldq, q_off, rows, heads, window, ring, row_pos, row_slot,
                 static_cast<const __nv_bfloat16*>(win), static_cast<const __nv_bfloat16*>(comp_pool), sel, n_sel, k,
                 page_table, max_pages, page_rows, inv_freq, rope_dim, scale, n_splits, row_hi, part_o, part_ml,
                 kv_row_bytes, row_lo, comp_row_bytes};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (D == 512) e = launch_attend<512>(p, s);
  else if (D == 128) e = launch_attend<128>(p, s);
  else return cudaErrorInvalidValue;
  if (e != cudaSuccess) return e;
  MergeParams m{part_o, part_ml, sink, row_pos, row_slot, inv_freq, rope_dim, heads, D, n_splits,
                static_cast<__nv_bfloat16*>(out), ldo};
  return launch_pdl(attend_merge_kernel, dim3(heads, rows), dim3(128), 0, s, m);
}
