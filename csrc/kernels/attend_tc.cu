// Sparse latent attention on the fifth-generation tensor cores (tcgen05 + TMEM).
//
// One CTA = one query row x all heads of this rank (MQA: every head reads the same latent rows, K == V), so a
// gathered key tile is fetched once and multiplied against all heads:  S = Q K^T  is one M=64 (heads) x N=64 (keys)
// accumulator in tensor memory, the softmax warps read it with tcgen05.ld, write P (bf16) back to shared memory in the
// UMMA-canonical 128-byte swizzle, and  O += P V  accumulates in tensor memory with the key tile as an MN-major B
// operand: the tile is stored once and serves as K (contracting D) and as V (contracting the keys).
//
// Tensor memory: an M=64 accumulator occupies lanes 0-15 of each 32-lane quadrant, so the two halves of a D=512 output
// row share 256 columns (second half at lane offset 16); two S buffers sit behind them.  Warp roles: 0-3 softmax,
// correction and epilogue (quadrant w = heads 16w..16w+15), 4-7 gather the key rows (window ring rows, then the
// selected compressed rows through the page table; bf16 rows by cp.async, FP8 / FP4 rows expanded in registers), 8
// issues the MMAs in whichever order their inputs arrive.  Keys are split across CTAs for decode-sized passes (partials
// merged by attend_merge_kernel); with one split the epilogue applies the sink, the normalisation and the inverse
// RoPE itself and writes bf16 rows.
//
// Semantics: native/cuda/kernels/v41_sparse_attention.cu:89-381 and native/cuda/kernels/v41_dspark_attention.cu:22-131
// of the reference (window + selected rows, per-head sink logit, optional window floor, drafter rows that see later
// rows of their block).  Every wait is bounded and reports through the status word.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"
#include "ds41_tma.h"

namespace ds41 {

constexpr int kTcHeads = 64;       // M of every MMA (heads of this rank, zero padded)
constexpr int kTcKeys = 64;        // keys per tile
constexpr int kTcThreads = 288;    // warps 0-3 softmax / epilogue, 4-7 gather, 8 MMA issue + TMEM owner
constexpr int kPanelBytes = 64 * 128;   // 64 rows (heads or keys) of one 128-byte swizzle span (64 bf16)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.f;     // the softmax reference moves only when a row maximum exceeds it by 2^8

struct AttendTcParams {
  const __nv_bfloat16* q;
  long long ldq;
  int q_off;
  int rows, heads, window, ring;
  const int* row_pos;
  const int* row_slot;
  const int* row_hi;
  const int* row_lo;
  const uint8_t* win;
  const uint8_t* comp_pool;
  const int* sel;
  const int* n_sel;
  int k;
  const int* page_table;
  int max_pages, page_rows;
  const float* inv_freq;
  int rope_dim;
  float scale;
  int n_splits;
  float* part_o;
  float* part_ml;
  const float* sink;
  __nv_bfloat16* out;
  long long ldo;
  int kv_row_bytes, comp_row_bytes;
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void rope_cs_tc(int pos, float inv_freq, float* c, float* s) {
  const double a = static_cast<double>(pos) * static_cast<double>(inv_freq);
  const double two_pi = 6.283185307179586476925286766559;
  const double red = a - floor(a * 0.15915494309189533576888376337251) * two_pi;
  sincosf(static_cast<float>(red), s, c);
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_drain() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void st_shared16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// byte offset of 16-byte chunk `ch` (8 bf16) of row `row` inside a tile stored as D/64 panels of [64 rows][128 B]
// 16 E4M3 values (one UE8M0 scale: a power of two, so the products are exact) -> 16 bf16 in two 16-byte chunks.
__device__ __forceinline__ void expand_fp8x16(const uint4& raw, uint32_t scale_e8m0, uint4& o0, uint4& o1) {
  const float sc = __uint_as_float(scale_e8m0 ? scale_e8m0 << 23 : 0x00400000u);     // 2^(e - 127); e = 0 is 2^-127
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_fp8x2_storage_t pair = static_cast<__nv_fp8x2_storage_t>((w[i >> 1] >> (16 * (i & 1))) & 0xffffu);
    const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3)));
    const __nv_bfloat162 v = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    o[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  o0 = make_uint4(o[0], o[1], o[2], o[3]);
  o1 = make_uint4(o[4], o[5], o[6], o[7]);
}

// 16 E2M1 values (8 bytes, low nibble first; one E4M3 scale) -> 16 bf16.  Magnitudes come from two byte tables through
// the byte-permute unit (the three magnitude bits of four values select four table bytes at once), the signs from its
// sign-replication mode; a value has at most 2 significant bits and the scale 4, so the bf16 products are exact.
__device__ __forceinline__ void expand_fp4x16(uint32_t x, uint32_t y, uint32_t scale_e4m3, uint4& o0, uint4& o1) {
  const __half_raw hs = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(scale_e4m3 & 0xffu), __NV_E4M3);
  const __nv_bfloat162 sc2 = __float2bfloat162_rn(__half2float(__half(hs)));
  const uint32_t in[2] = {x, y};
  uint32_t o[8];
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const uint32_t word = in[h >> 1], word4 = word << 4;
    const uint32_t sel = ((h & 1) ? word >> 16 : word) & 0x7777u;
    const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, sel);     // low bytes of bf16 {0, .5, 1, 1.5, 2, 3, 4, 6}
    const uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);     // high bytes
    uint32_t w0 = __byte_perm(lo, hi, 0x5140u), w1 = __byte_perm(lo, hi, 0x7362u);
    // bit 15 / 31 of a pair <- sign nibble bits of its two values (most significant bit of a byte of word << 4 / word)
    const uint32_t m0 = __byte_perm(word4, word, (h & 1) ? 0xE0A0u : 0xC080u);
    const uint32_t m1 = __byte_perm(word4, word, (h & 1) ? 0xF0B0u : 0xD090u);
    w0 ^= m0 & 0x80008000u;
    w1 ^= m1 & 0x80008000u;
    const __nv_bfloat162 v0 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w0), sc2);
    const __nv_bfloat162 v1 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w1), sc2);
    o[2 * h] = *reinterpret_cast<const uint32_t*>(&v0);
    o[2 * h + 1] = *reinterpret_cast<const uint32_t*>(&v1);
  }
  o0 = make_uint4(o[0], o[1], o[2], o[3]);
  o1 = make_uint4(o[4], o[5], o[6], o[7]);
}

__device__ __forceinline__ uint32_t tile_off(int row, int ch) {
  return static_cast<uint32_t>((ch >> 3) * kPanelBytes + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
}

// Debug builds (-DDS41_ATTN_TRACE) record clock64 stamps of CTA 0's pipeline events in a global buffer.
#ifdef DS41_ATTN_TRACE
__device__ long long ds41_attn_trace[4][4096];
#define ATTN_TRACE(role, idx, code)                                                                  \
  do {                                                                                               \
    if (blockIdx.x == 0 && (idx) < 2047) {                                                           \
      ds41_attn_trace[role][2 * (idx)] = (code);                                                     \
      ds41_attn_trace[role][2 * (idx) + 1] = clock64();                                              \
    }                                                                                                \
  } while (0)
#else
#define ATTN_TRACE(role, idx, code) do { } while (0)
#endif

template <int D>
struct AttendTcCfg {
  static constexpr int kPanels = D / 64;
  static constexpr int kTile = kPanels * kPanelBytes;                 // one Q or K tile
  static constexpr int kOCols = D >= 256 ? 256 : D;                   // accumulator columns per half of D
  static constexpr int kHalves = D / kOCols;
  static constexpr int kSCol = kOCols;                                // first S buffer
  static constexpr int kSBuf = 2 * kTcKeys;                           // one S buffer: two partial accumulators
  static constexpr int kTmemCols = kOCols + 2 * kSBuf <= 256 ? 256 : 512;
  static_assert(kOCols + 2 * kSBuf <= 512, "tensor memory budget");
  static constexpr int kSmem = 1024 + 3 * kTile + 2 * kPanelBytes + 8 * 2 * 64 * 4 + 16 * 8 + 64;
  static_assert(D % 64 == 0 && kHalves <= 2, "head width");
};

// What one work item (a query row and one split of its key tiles) covers; every role derives it the same way.
struct ItemShape {
  int r, split, pos, slot, lo_pos, n_w, n_keys, n_my;
};
__device__ __forceinline__ ItemShape item_shape(const AttendTcParams& p, int item) {
  ItemShape s;
  s.r = item / p.n_splits;
  s.split = item - s.r * p.n_splits;
  s.pos = p.row_pos[s.r];
  s.slot = p.row_slot[s.r];
  s.lo_pos = 0;
  s.n_w = 0;
  int n_s = 0;
  if (s.slot >= 0) {
    int hi_pos = s.pos;
    if (p.row_hi != nullptr) hi_pos = max(s.pos, p.row_hi[s.r]);    // drafter rows see later rows of their block
    s.lo_pos = max(0, s.pos - p.window + 1);
    if (p.row_lo != nullptr) s.lo_pos = max(s.lo_pos, p.row_lo[s.r]);
    s.n_w = max(0, hi_pos - s.lo_pos + 1);
    n_s = (p.comp_pool != nullptr && p.n_sel != nullptr) ? p.n_sel[s.r] : 0;
  }
  s.n_keys = s.n_w + n_s;
  const int n_tiles = (s.n_keys + kTcKeys - 1) / kTcKeys;
  s.n_my = s.split < n_tiles ? (n_tiles - s.split + p.n_splits - 1) / p.n_splits : 0;
  return s;
}

// Persistent kernel: CTA c takes the work items c, c + gridDim.x, ...  Tensor memory, the barriers and the shared
// memory tiles are set up once; tiles are counted through all items of a CTA (buffer = count & 1, barrier parity =
// (count >> 1) & 1), items that have keys are counted separately for the per-item barriers.
template <int D>
__global__ void __launch_bounds__(kTcThreads, 1) attend_tc_kernel(AttendTcParams p) {
  using Cfg = AttendTcCfg<D>;
  constexpr int CH = D / 8;                    // 16-byte chunks per bf16 row
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTile;               // [2][kTile]
  uint8_t* sP = sK + 2 * Cfg::kTile;           // [2][kPanelBytes]
  float* sTrig = reinterpret_cast<float*>(sP + 2 * kPanelBytes);  // [8 warps][cos 64 | sin 64], private to each warp
  uint64_t* k_full = reinterpret_cast<uint64_t*>(sTrig + 8 * 128);   // [2] gather -> MMA
  uint64_t* k_free = k_full + 2;               // [2] MMA -> gather / correction: P V of the tile in this buffer is done
  uint64_t* s_full = k_free + 2;               // [2] MMA -> softmax
  uint64_t* p_full = s_full + 2;               // [2] softmax -> MMA
  uint64_t* q_full = p_full + 2;               // gather -> MMA: the item's Q tile is in place
  uint64_t* q_free = q_full + 1;               // MMA -> gather: the item's last S has read the Q tile
  uint64_t* o_full = q_free + 1;               // MMA -> epilogue: the item's last P V is done
  uint64_t* o_free = o_full + 1;               // epilogue -> MMA: the accumulators have been read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_heads = min(kTcHeads, p.heads);
  const int n_items = p.rows * p.n_splits;
  const bool final_out = p.n_splits == 1;
  pdl_launch_dependents();

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&k_full[b], 4);
      mbar_init(&k_free[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4);
    }
    mbar_init(q_full, 4);
    mbar_init(q_free, 1);
    mbar_init(o_full, 1);
    mbar_init(o_free, 4);
    mbar_init_fence();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------ gather: Q rows and 16 keys of every tile per warp
    const int lw = warp - 4;
    float* my_cos = sTrig + warp * 128;
    float* my_sin = my_cos + 64;
    const long long row_bytes = p.kv_row_bytes > 0 ? p.kv_row_bytes : 2ll * D;
    const long long comp_bytes = p.comp_row_bytes > 0 ? p.comp_row_bytes : row_bytes;
    const int rope0 = D - p.rope_dim;
    const int n_plain = rope0 / 8;               // chunks per head that are copied as they are
    const uint32_t sq = smem_u32(sQ);
    // (item, tile) pairs with keys, in the order every role walks them
    auto next_tile = [&](int& item, ItemShape& s, int& j) -> bool {
      ++j;
      while (item < n_items && j >= s.n_my) {
        item += gridDim.x;
        j = 0;
        if (item < n_items) s = item_shape(p, item);
      }
      return item < n_items;
    };
    // address of key (16 lw + lane) of a tile, lanes 0-15; the two dependent loads behind a selected row are issued
    // one tile ahead of their use
    auto lookup = [&](const ItemShape& s, int j, const uint8_t*& ptr, int& fp4) {
      ptr = nullptr;
      fp4 = 0;
      if (lane >= 16) return;
      const int jk = (s.split + j * p.n_splits) * kTcKeys + lw * 16 + lane;
      if (jk >= s.n_keys) return;
      if (jk < s.n_w) {
        const int kp = s.lo_pos + jk;
        ptr = p.win + (1ll * s.slot * p.ring + (kp % p.ring)) * row_bytes;
        return;
      }
      const int id = p.sel[1ll * s.r * p.k + (jk - s.n_w)];
      if (id < 0) return;
      const int page = p.page_table[1ll * s.slot * p.max_pages + id / p.page_rows];
      if (page < 0) return;
      ptr = p.comp_pool + (1ll * page * p.page_rows + id % p.page_rows) * comp_bytes;
      fp4 = p.comp_row_bytes > 0 ? 1 : 0;
    };
    int item = static_cast<int>(blockIdx.x) - static_cast<int>(gridDim.x), j = 0;
    ItemShape s{};
    s.n_my = 0;
    bool live = next_tile(item, s, j);
    const uint8_t* my_ptr = nullptr;
    int my_fp4 = 0;
    if (live) lookup(s, j, my_ptr, my_fp4);
    bool ok = true;
    int g = 0, it = 0;                           // tiles / items with keys so far
    while (live && ok) {
      if (j == 0) {
        // ---- Q tile of this row: heads [16 lw, 16 lw + 16); RoPE on the tail, zero rows for heads this rank lacks
        if (lane < p.rope_dim / 2) rope_cs_tc(s.pos, p.inv_freq[lane], &my_cos[lane], &my_sin[lane]);
        if (lane + 32 < p.rope_dim / 2) rope_cs_tc(s.pos, p.inv_freq[lane + 32], &my_cos[lane + 32], &my_sin[lane + 32]);
        if (it >= 1) {
          ok = mbar_wait(q_free, (it - 1) & 1, p.status, 401);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        __syncwarp();
        const __nv_bfloat16* qrow = p.q + 1ll * s.r * p.ldq + p.q_off;
        for (int idx = lane; idx < 16 * n_plain; idx += 32) {
          const int h = lw * 16 + idx / n_plain, ch = idx % n_plain;
          if (h < n_heads) cp_async16(sq + tile_off(h, ch), qrow + 1ll * h * D + ch * 8);
          else st_shared16(sq + tile_off(h, ch), make_uint4(0, 0, 0, 0));
        }
        // rotary chunks pass through registers, four at a time: all their loads are in flight before the first use
        const int n_rot = 16 * (CH - n_plain);
        for (int i0 = lane; i0 < n_rot; i0 += 128) {
          uint4 raw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int idx = i0 + 32 * u;
            const int h = lw * 16 + idx / (CH - n_plain), ch = n_plain + idx % (CH - n_plain);
            raw[u] = make_uint4(0, 0, 0, 0);
            if (idx < n_rot && h < n_heads) raw[u] = __ldg(reinterpret_cast<const uint4*>(qrow + 1ll * h * D + ch * 8));
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int idx = i0 + 32 * u;
            if (idx >= n_rot) continue;
            const int h = lw * 16 + idx / (CH - n_plain), ch = n_plain + idx % (CH - n_plain);
            __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw[u]);
#pragma unroll
            for (int q2 = 0; q2 < 4; ++q2) {
              const float2 f = __bfloat1622float2(v[q2]);
              const int t = (ch * 8 + 2 * q2 - rope0) / 2;
              const float c = my_cos[t], sn = my_sin[t];
              v[q2] = __floats2bfloat162_rn(f.x * c - f.y * sn, f.y * c + f.x * sn);
            }
            st_shared16(sq + tile_off(h, ch), raw[u]);
          }
        }
      }
      const int b = g & 1;
      if (g >= 2) {
        ok = mbar_wait(&k_free[b], ((g >> 1) - 1) & 1, p.status, 400);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (lw == 0 && lane == 0) ATTN_TRACE(0, 3 * g, 10 + b);
      const uint32_t kb = smem_u32(sK + b * Cfg::kTile);
      const uint32_t null_mask = __ballot_sync(0xffffffffu, my_ptr == nullptr) & 0xffffu;
      const uint32_t fp4_mask = __ballot_sync(0xffffffffu, my_fp4 != 0) & 0xffffu;
      if (p.kv_row_bytes == 0) {
        // bf16 rows: asynchronous 16-byte copies straight into the swizzled tile.  Lane l copies chunks l, l + 32, ...
        // of every key; only the row term and the swizzle's XOR change from key to key (compile-time here).
        const uint32_t dst_lane = kb + (lane >> 3) * kPanelBytes + lw * 16 * 128;
        const uint32_t x_lane = (lane & 7) << 4;
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(
              __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_ptr), kk));
          const uint32_t dst = dst_lane + kk * 128 + (x_lane ^ ((kk & 7) << 4));
          if (src == nullptr) {
#pragma unroll
            for (int i = 0; i < (CH + 31) / 32; ++i)
              if (lane + 32 * i < CH) st_shared16(dst + i * 4 * kPanelBytes, make_uint4(0, 0, 0, 0));
          } else {
            src += lane * 16;
#pragma unroll
            for (int i = 0; i < (CH + 31) / 32; ++i)
              if (lane + 32 * i < CH) cp_async16(dst + i * 4 * kPanelBytes, src + i * 512);
          }
        }
      } else {
        // quantised rows.  Lane u expands values [16u, 16u + 16) of every key - 16 bytes of an FP8 row (one UE8M0
        // scale per 32 values behind the D values) or 8 bytes of an FP4 row (one E4M3 scale per 16 values behind the
        // D/2 bytes) - into the two 16-byte chunks 2u, 2u + 1 of the key's tile row.  Keys pass through registers four
        // at a time, the next four loads in flight while the current four are expanded.  The loop over the groups
        // stays rolled: unrolled over 16 keys its code does not fit the instruction cache and every tile refetches it.
        const bool act = lane < D / 16;
        uint4 nxt[4];
        uint32_t nsc[4];
        auto load4 = [&](int grp) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int kk = 4 * grp + u;
            const uint8_t* src = reinterpret_cast<const uint8_t*>(
                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_ptr), kk));
            nxt[u] = make_uint4(0, 0, 0, 0);
            nsc[u] = 0;
            if (src != nullptr && act) {
              if ((fp4_mask >> kk) & 1u) {
                const uint2 t = __ldg(reinterpret_cast<const uint2*>(src + lane * 8));
                nxt[u].x = t.x;
                nxt[u].y = t.y;
                nsc[u] = __ldg(src + D / 2 + lane);
              } else {
                nxt[u] = __ldg(reinterpret_cast<const uint4*>(src + lane * 16));
                nsc[u] = __ldg(src + D + (lane >> 1));
              }
            }
          }
        };
        load4(0);
#pragma unroll 1
        for (int grp = 0; grp < 4; ++grp) {
          uint4 cur[4];
          uint32_t csc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) { cur[u] = nxt[u]; csc[u] = nsc[u]; }
          if (grp < 3) load4(grp + 1);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int kk = 4 * grp + u, key = lw * 16 + kk;
            uint4 o0 = make_uint4(0, 0, 0, 0), o1 = o0;
            if (!((null_mask >> kk) & 1u)) {
              if ((fp4_mask >> kk) & 1u) expand_fp4x16(cur[u].x, cur[u].y, csc[u], o0, o1);
              else expand_fp8x16(cur[u], csc[u], o0, o1);
            }
            if (act) {
              st_shared16(kb + tile_off(key, 2 * lane), o0);
              st_shared16(kb + tile_off(key, 2 * lane + 1), o1);
            }
          }
        }
      }
      if (lw == 0 && lane == 0) ATTN_TRACE(0, 3 * g + 1, 20 + b);
      // the next tile's addresses are looked up while this tile's copies land
      const bool first_of_item = j == 0;
      const int item_before = item;
      live = next_tile(item, s, j);
      if (live) lookup(s, j, my_ptr, my_fp4);
      cp_async_drain();                         // covers the Q copies on the item's first tile
      if (lw == 0 && lane == 0) ATTN_TRACE(0, 3 * g + 2, 30 + b);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (first_of_item) mbar_arrive(q_full);
        mbar_arrive(&k_full[b]);
      }
      ++g;
      if (!live || item != item_before) ++it;
    }
    cp_async_drain();
  } else if (warp == 8) {
    // ------------------------------------------------------------ MMA issue
    // The whole warp walks the loop (its branches are warp-uniform at run time); `leader` predicates the tensor-core
    // instructions themselves.  The two buffers have their own unrolled copies so that every descriptor is a
    // loop-invariant base plus a compile-time offset.
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = umma_idesc(kTcHeads, kTcKeys, 1u, 1u);
    constexpr uint32_t idesc_pv = umma_idesc_bmn(kTcHeads, Cfg::kOCols, 1u, 1u);
    const uint64_t q_desc = umma_desc_sw128(smem_u32(sQ));
    const uint64_t k_desc0 = umma_desc_sw128(smem_u32(sK)), k_desc1 = umma_desc_sw128(smem_u32(sK) + Cfg::kTile);
    const uint64_t p_desc0 = umma_desc_sw128(smem_u32(sP)), p_desc1 = umma_desc_sw128(smem_u32(sP) + kPanelBytes);
    const uint64_t v_desc0 = umma_desc_sw128_mn(smem_u32(sK), kPanelBytes, 1024);
    const uint64_t v_desc1 = umma_desc_sw128_mn(smem_u32(sK) + Cfg::kTile, kPanelBytes, 1024);
    // S = Q K^T of one tile.  Consecutive MMAs into one accumulator wait for each other: even and odd 16-wide slices
    // of D go to two accumulators, which the softmax warps add.
    auto issue_s = [&](uint32_t s_tmem, uint64_t kd) {
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        constexpr int kPanel16 = kPanelBytes / 16;
        const uint64_t off = static_cast<uint64_t>((k >> 2) * kPanel16 + (k & 3) * 2);
        umma_bf16_if(leader, s_tmem + (k & 1) * kTcKeys, q_desc + off, kd + off, idesc_s, k > 1 ? 1u : 0u);
      }
    };
    // O (+)= P V of one tile: the key tile as an MN-major operand, one accumulator per half of D
    auto issue_pv = [&](uint64_t pd, uint64_t vd, uint32_t first) {
#pragma unroll
      for (int ks = 0; ks < kTcKeys / 16; ++ks) {
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) {
          const uint64_t voff = static_cast<uint64_t>((h * (Cfg::kOCols / 64) * kPanelBytes + ks * 2048) / 16);
          umma_bf16_if(leader, tmem_base + (static_cast<uint32_t>(h * 16) << 16), pd + static_cast<uint64_t>(ks * 2),
                       vd + voff, idesc_pv, ks > 0 ? 1u : first);
        }
      }
    };
    int g0 = 0, it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const ItemShape s = item_shape(p, item);
      if (s.n_my == 0) continue;
      ok = mbar_wait(q_full, it & 1, p.status, 411);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      int next_s = 0, next_pv = 0;
      long long start = clock64();
      uint32_t spins = 0;
      while (next_pv < s.n_my) {
        bool progressed = false;
        if (next_s < s.n_my && next_s < next_pv + 2) {
          const int g = g0 + next_s, b = g & 1;
          if (__all_sync(0xffffffffu, mbar_test_wait(&k_full[b], (g >> 1) & 1))) {
            if (leader) ATTN_TRACE(1, 2 * g, 100 + b);
            tc_fence_after();
            if (b == 0) issue_s(tmem_base + Cfg::kSCol, k_desc0);
            else issue_s(tmem_base + Cfg::kSCol + Cfg::kSBuf, k_desc1);
            tc_commit_if(leader, &s_full[b]);
            if (next_s == s.n_my - 1) tc_commit_if(leader, q_free);
            ++next_s;
            progressed = true;
          }
        }
        if (next_pv < next_s) {
          const int g = g0 + next_pv, b = g & 1;
          // the first product of an item overwrites the accumulators: the previous item's epilogue must have read them
          const bool o_ready = next_pv > 0 || it == 0 || mbar_test_wait(o_free, (it - 1) & 1);
          if (__all_sync(0xffffffffu, o_ready && mbar_test_wait(&p_full[b], (g >> 1) & 1))) {
            if (leader) ATTN_TRACE(1, 2 * g + 1, 200 + b);
            tc_fence_after();
            const uint32_t first = next_pv > 0 ? 1u : 0u;
            if (b == 0) issue_pv(p_desc0, v_desc0, first);
            else issue_pv(p_desc1, v_desc1, first);
            tc_commit_if(leader, &k_free[b]);
            if (next_pv == s.n_my - 1) tc_commit_if(leader, o_full);
            ++next_pv;
            progressed = true;
          }
        }
        if (progressed) {
          start = clock64();
          spins = 0;
        } else if ((++spins & 0x3ff) == 0) {
          const bool give_up = clock64() - start > DS41_WAIT_LIMIT_CYCLES ||
                               (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != kStatusOk);
          if (__any_sync(0xffffffffu, give_up)) {
            if (leader && p.status != nullptr && atomicCAS(p.status, kStatusOk, kStatusMbarTimeout) == kStatusOk) {
              p.status[1] = 410;
              p.status[2] = s.r;
              p.status[3] = next_s * 1000 + next_pv;
            }
            ok = false;
            break;
          }
        }
      }
      g0 += s.n_my;
      ++it;
    }
  } else {
    // ------------------------------------------------------------ softmax, correction, epilogue (warps 0-3)
    const int hsel = lane & 15, half = lane >> 4;
    const int head = warp * 16 + hsel;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float scale2 = p.scale * kLog2e;
    const bool o_owner = half < Cfg::kHalves;         // lanes 16-31 hold the second half of D when it is interleaved
    float* my_cos = sTrig + warp * 128;
    float* my_sin = my_cos + 64;
    const int rope0 = D - p.rope_dim;
    // epilogue staging: this warp's own rows of the two P buffers (16 rows x 128 B each), idle once the item's last
    // product has run: lanes 0-15 stage half 0 in buffer 0, lanes 16-31 half 1 in buffer 1
    const uint32_t stage_row = smem_u32(sP) + half * kPanelBytes + (warp * 16 + hsel) * 128;
    const uint8_t* stage_base = sP + warp * 16 * 128;
    bool ok = true;
    int g = 0, it = 0;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const ItemShape s = item_shape(p, item);
      if (s.n_my == 0) {
        if (final_out) {
          // a row without keys (a padding row): zeros
          for (int i = tid; i < n_heads * CH; i += 128)
            *reinterpret_cast<uint4*>(p.out + 1ll * s.r * p.ldo + 8ll * i) = make_uint4(0, 0, 0, 0);
        } else if (tid < n_heads) {
          float* ml = p.part_ml + ((1ll * s.r * p.n_splits + s.split) * p.heads + tid) * 2;
          ml[0] = -INFINITY;
          ml[1] = 0.f;
        }
        continue;
      }
      if (final_out) {
        // inverse-rotation table of this row, private to the warp (read in the epilogue)
        if (lane < p.rope_dim / 2) rope_cs_tc(s.pos, p.inv_freq[lane], &my_cos[lane], &my_sin[lane]);
        if (lane + 32 < p.rope_dim / 2) rope_cs_tc(s.pos, p.inv_freq[lane + 32], &my_cos[lane + 32], &my_sin[lane + 32]);
        __syncwarp();
      }
      float m_ref = -INFINITY, l = 0.f;               // per head (lanes 0-15), in log2 units
      for (int j = 0; j < s.n_my && ok; ++j, ++g) {
        const int tile = s.split + j * p.n_splits;
        const int b = g & 1;
        const int k_cnt = min(kTcKeys, s.n_keys - tile * kTcKeys);
        ok = mbar_wait(&s_full[b], (g >> 1) & 1, p.status, 420);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (warp == 0 && lane == 0) ATTN_TRACE(2, 3 * g, 300 + b);
        uint32_t v0[32], v1[32];
        {
          // S = the sum of the two partial accumulators
          uint32_t u[32];
          const uint32_t s_tmem = t_lane + Cfg::kSCol + Cfg::kSBuf * b;
          tmem_ld_32x32(s_tmem, v0);
          tmem_ld_32x32(s_tmem + kTcKeys, u);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) v0[c] = __float_as_uint(__uint_as_float(v0[c]) + __uint_as_float(u[c]));
          tmem_ld_32x32(s_tmem + 32, v1);
          tmem_ld_32x32(s_tmem + kTcKeys + 32, u);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) v1[c] = __float_as_uint(__uint_as_float(v1[c]) + __uint_as_float(u[c]));
        }
        if (warp == 0 && lane == 0) ATTN_TRACE(2, 3 * g + 1, 310 + b);
        if (k_cnt < kTcKeys) {
          // the row's last tile: columns beyond its keys take no part
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c >= k_cnt) v0[c] = 0xff800000u;
            if (c + 32 >= k_cnt) v1[c] = 0xff800000u;
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[c]), __uint_as_float(v1[c])));
        mx *= scale2;                                 // scale2 > 0
        const bool need = lane < 16 && mx > m_ref + kRescaleStep;
        if (__any_sync(0xffffffffu, need)) {
          // the reference of every head of this quadrant moves to its running maximum; O and l follow
          const float m_new = fmaxf(m_ref, mx);
          const float alpha = m_ref == -INFINITY ? 0.f : ex2(m_ref - m_new);
          l *= alpha;
          m_ref = m_new;
          if (j > 0) {
            const float a_o = __shfl_sync(0xffffffffu, alpha, hsel);
            ok = mbar_wait(&k_free[(g - 1) & 1], ((g - 1) >> 1) & 1, p.status, 421);     // P V of the previous tile
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c0 = 0; c0 < Cfg::kOCols; c0 += 32) {
              uint32_t o[32];
              tmem_ld_32x32(t_lane + c0, o);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * a_o);
              tmem_st_32x32(t_lane + c0, o);
            }
            tmem_wait_st();
          }
        }
        // P = 2^(s * scale - reference) in bf16; the row sum adds the rounded values (what the tensor core multiplies)
        const float neg_m = -m_ref;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const __nv_bfloat162 e = __floats2bfloat162_rn(ex2(fmaf(__uint_as_float(v0[c]), scale2, neg_m)),
                                                         ex2(fmaf(__uint_as_float(v0[c + 1]), scale2, neg_m)));
          const __nv_bfloat162 f = __floats2bfloat162_rn(ex2(fmaf(__uint_as_float(v1[c]), scale2, neg_m)),
                                                         ex2(fmaf(__uint_as_float(v1[c + 1]), scale2, neg_m)));
          const uint32_t eu = *reinterpret_cast<const uint32_t*>(&e), fu = *reinterpret_cast<const uint32_t*>(&f);
          sum0 += __uint_as_float(eu << 16) + __uint_as_float(eu & 0xffff0000u);
          sum1 += __uint_as_float(fu << 16) + __uint_as_float(fu & 0xffff0000u);
          pk[c >> 1] = eu;
          pk[16 + (c >> 1)] = fu;
        }
        l += sum0 + sum1;
        if (lane < 16) {
          const uint32_t prow = smem_u32(sP + b * kPanelBytes) + head * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared16(prow + ((c ^ (head & 7)) << 4), make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]));
        }
        tc_fence_before();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[b]);
        if (warp == 0 && lane == 0) ATTN_TRACE(2, 3 * g + 2, 320 + b);
      }
      if (ok) ok = mbar_wait(o_full, it & 1, p.status, 430);
      if (warp == 0 && lane == 0) ATTN_TRACE(3, 2 * it, 400);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float l_h = __shfl_sync(0xffffffffu, l, hsel);
      const float m_h = __shfl_sync(0xffffffffu, m_ref, hsel);
      float f = 1.f;
      if (final_out) {
        const float sink2 = (head < n_heads ? __ldg(p.sink + head) : 0.f) * kLog2e;
        const float m_fin = fmaxf(m_h, sink2);
        const float w_o = ex2(m_h - m_fin);
        f = w_o / (l_h * w_o + ex2(sink2 - m_fin));
      } else if (lane < 16 && head < n_heads) {
        float* ml = p.part_ml + ((1ll * s.r * p.n_splits + s.split) * p.heads + head) * 2;
        ml[0] = m_h / kLog2e;
        ml[1] = l_h;
      }
      // Rounds of 128 bytes per (head, half of D): every lane stages its row's piece in shared memory, then the warp
      // writes the staged rows, four per instruction (lane l moves 16-byte chunk l & 7 of row l >> 3).  The accumulator
      // columns of the next round are fetched from tensor memory before the current round is processed.
      const int heads_here = max(0, min(16, n_heads - warp * 16));      // this warp's heads that exist
      auto release_o = [&]() {
        // the accumulators are in registers: the next item's first product may overwrite them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free);
      };
      auto flush_rows = [&](auto* row0, int elems_per_chunk) {
        __syncwarp();
#pragma unroll
        for (int r0 = 0; r0 < 16 * Cfg::kHalves; r0 += 16) {
          uint4 val[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rr = r0 + 4 * i + (lane >> 3), hh = rr & 15, hf = rr >> 4;
            val[i] = *reinterpret_cast<const uint4*>(stage_base + hf * kPanelBytes + hh * 128 + (((lane & 7) ^ (hh & 7)) << 4));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rr = r0 + 4 * i + (lane >> 3), hh = rr & 15, hf = rr >> 4;
            if (hh < heads_here)
              *reinterpret_cast<uint4*>(row0 + 1ll * (warp * 16 + hh) * D + hf * Cfg::kOCols + elems_per_chunk * (lane & 7)) = val[i];
          }
        }
        __syncwarp();
      };
      if (final_out) {
        __nv_bfloat16* orow = p.out + 1ll * s.r * p.ldo;
        constexpr int kRounds = Cfg::kOCols / 64;
        uint32_t oa[2][32], ob[2][32];                 // two rounds of 64 columns in flight
        tmem_ld_32x32(t_lane, oa[0]);
        tmem_ld_32x32(t_lane + 32, ob[0]);
#pragma unroll
        for (int rd = 0; rd < kRounds; ++rd) {
          const int c0 = rd * 64;
          tmem_wait_ld();
          if (rd + 1 < kRounds) {
            tmem_ld_32x32(t_lane + c0 + 64, oa[(rd + 1) & 1]);
            tmem_ld_32x32(t_lane + c0 + 96, ob[(rd + 1) & 1]);
          } else {
            release_o();
          }
          const uint32_t* o0 = oa[rd & 1];
          const uint32_t* o1 = ob[rd & 1];
          const int d0 = half * Cfg::kOCols + c0;
          uint32_t w[32];
          if (d0 + 64 > rope0) {
            // this round reaches into the rotary tail: inverse rotation of the pairs at or above rope0
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
              float a = __uint_as_float(c < 32 ? o0[c] : o1[c - 32]) * f;
              float bb = __uint_as_float(c < 32 ? o0[c + 1] : o1[c - 31]) * f;
              const int t = d0 + c - rope0;
              if (t >= 0) {
                const float cs = my_cos[t >> 1], sn = my_sin[t >> 1];
                const float ra = a * cs + bb * sn, rb = bb * cs - a * sn;
                a = ra;
                bb = rb;
              }
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, bb);
              w[c >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(c < 32 ? o0[c] : o1[c - 32]) * f,
                                                              __uint_as_float(c < 32 ? o0[c + 1] : o1[c - 31]) * f);
              w[c >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
            }
          }
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared16(stage_row + ((c ^ (hsel & 7)) << 4), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
          flush_rows(orow + c0, 8);
        }
      } else {
        float* prow = p.part_o + (1ll * s.r * p.n_splits + s.split) * p.heads * D;
        constexpr int kRounds = Cfg::kOCols / 32;
        uint32_t oa[2][32];
        tmem_ld_32x32(t_lane, oa[0]);
#pragma unroll
        for (int rd = 0; rd < kRounds; ++rd) {
          const int c0 = rd * 32;
          tmem_wait_ld();
          if (rd + 1 < kRounds) tmem_ld_32x32(t_lane + c0 + 32, oa[(rd + 1) & 1]);
          else release_o();
          const uint32_t* o = oa[rd & 1];
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared16(stage_row + ((c ^ (hsel & 7)) << 4), make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
          flush_rows(prow + c0, 4);
        }
      }
      if (warp == 0 && lane == 0) ATTN_TRACE(3, 2 * it + 1, 410);
      ++it;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != kStatusOk) {
    // a wait gave up: let copies and MMAs that may still be in flight finish before the CTA's memory goes away
    const long long start = clock64();
    while (clock64() - start < 2000000ll) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 8) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int D>
static cudaError_t launch_attend_tc(const AttendTcParams& p, cudaStream_t stream) {
  using Cfg = AttendTcCfg<D>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attend_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const long long items = 1ll * p.rows * p.n_splits;
  const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
  return launch_pdl(attend_tc_kernel<D>, dim3(grid), dim3(kTcThreads), Cfg::kSmem, stream, p);
}

}  // namespace ds41

using namespace ds41;

#ifdef DS41_ATTN_TRACE
extern "C" int ds41_attn_trace_read(long long* host, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(host, ds41_attn_trace, sizeof(long long) * 4 * 4096);
  if (e != cudaSuccess) return e;
  if (clear) {
    static long long zeros[4 * 4096];
    e = cudaMemcpyToSymbol(ds41_attn_trace, zeros, sizeof(zeros));
  }
  return e;
}
#endif

extern "C" int ds41_attend_tc(const ds41_attend_args* a, void* stream) {
  if (a == nullptr || a->rows <= 0 || a->heads <= 0 || a->heads > kTcHeads || a->n_splits <= 0 || a->n_splits > 32 ||
      a->rope_dim > 128 || (a->rope_dim & 7) || a->rope_dim > a->D || a->q == nullptr || a->win == nullptr ||
      a->row_pos == nullptr || a->row_slot == nullptr || a->inv_freq == nullptr || a->sink == nullptr ||
      a->out == nullptr || (a->ldq & 7) || (a->q_off & 7) || (a->ldo & 7))
    return cudaErrorInvalidValue;
  if (a->n_splits > 1 && (a->part_o == nullptr || a->part_ml == nullptr)) return cudaErrorInvalidValue;
  if (a->kv_row_bytes != 0 && (a->kv_row_bytes < a->D + a->D / 32 || (a->kv_row_bytes & 15))) return cudaErrorInvalidValue;
  if (a->comp_row_bytes != 0 && (a->kv_row_bytes <= 0 || a->comp_row_bytes < a->D / 2 + a->D / 16 || (a->comp_row_bytes & 15)))
    return cudaErrorInvalidValue;
  if (a->comp_pool != nullptr && (a->sel == nullptr || a->n_sel == nullptr || a->page_table == nullptr || a->page_rows <= 0))
    return cudaErrorInvalidValue;
  AttendTcParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.ldq = a->ldq; p.q_off = a->q_off;
  p.rows = a->rows; p.heads = a->heads; p.window = a->window; p.ring = a->ring;
  p.row_pos = a->row_pos; p.row_slot = a->row_slot; p.row_hi = a->row_hi; p.row_lo = a->row_lo;
  p.win = static_cast<const uint8_t*>(a->win);
  p.comp_pool = static_cast<const uint8_t*>(a->comp_pool);
  p.sel = a->sel; p.n_sel = a->n_sel; p.k = a->k;
  p.page_table = a->page_table; p.max_pages = a->max_pages; p.page_rows = a->page_rows;
  p.inv_freq = a->inv_freq; p.rope_dim = a->rope_dim; p.scale = a->scale;
  p.n_splits = a->n_splits; p.part_o = a->part_o; p.part_ml = a->part_ml; p.sink = a->sink;
  p.out = static_cast<__nv_bfloat16*>(a->out); p.ldo = a->ldo;
  p.kv_row_bytes = a->kv_row_bytes; p.comp_row_bytes = a->comp_row_bytes;
  p.status = a->status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (a->D == 512) e = launch_attend_tc<512>(p, s);
  else if (a->D == 128) e = launch_attend_tc<128>(p, s);
  else return cudaErrorInvalidValue;
  if (e != cudaSuccess || a->n_splits == 1) return e;
  return ds41_attend_merge(a->part_o, a->part_ml, a->sink, a->row_pos, a->row_slot, a->inv_freq, a->rope_dim, a->heads,
                           a->D, a->n_splits, a->rows, a->out, a->ldo, stream);
}
