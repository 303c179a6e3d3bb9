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
  int split_d;
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
__device__ __forceinline__ uint32_t tile_off(int row, int ch) {
  return static_cast<uint32_t>((ch >> 3) * kPanelBytes + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
}

template <int D>
struct AttendTcCfg {
  static constexpr int kPanels = D / 64;
  static constexpr int kTile = kPanels * kPanelBytes;                 // one Q or K tile
  static constexpr int kOCols = D >= 256 ? 256 : D;                   // accumulator columns per half of D
  static constexpr int kHalves = D / kOCols;
  static constexpr int kSCol = kOCols;                                // first S buffer
  static constexpr int kTmemCols = kOCols + 2 * kTcKeys <= 256 ? 256 : 512;
  static constexpr int kSmem = 1024 + 3 * kTile + 2 * kPanelBytes + 2 * 64 * 4 + 16 * 8 + 64;
  static_assert(D % 64 == 0 && kHalves <= 2, "head width");
};

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
  float* sCos = reinterpret_cast<float*>(sP + 2 * kPanelBytes);   // [64]
  float* sSin = sCos + 64;
  uint64_t* k_full = reinterpret_cast<uint64_t*>(sSin + 64);      // [2] gather -> MMA
  uint64_t* k_free = k_full + 2;               // [2] MMA -> gather / correction: P V of the tile in this buffer is done
  uint64_t* s_full = k_free + 2;               // [2] MMA -> softmax
  uint64_t* p_full = s_full + 2;               // [2] softmax -> MMA
  uint64_t* o_full = p_full + 2;               // the last P V is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);

  const int split = blockIdx.x, r = blockIdx.y, dz = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_heads = min(kTcHeads, p.heads);
  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.row_pos[r], slot = p.row_slot[r];
  int n_w = 0, n_s = 0, lo_pos = 0;
  if (slot >= 0) {
    int hi_pos = pos;
    if (p.row_hi != nullptr) hi_pos = max(pos, p.row_hi[r]);      // drafter rows see later rows of their block
    lo_pos = max(0, pos - p.window + 1);
    if (p.row_lo != nullptr) lo_pos = max(lo_pos, p.row_lo[r]);
    n_w = max(0, hi_pos - lo_pos + 1);
    n_s = (p.comp_pool != nullptr && p.n_sel != nullptr) ? p.n_sel[r] : 0;
  }
  const int n_keys = n_w + n_s;
  const int n_tiles = (n_keys + kTcKeys - 1) / kTcKeys;
  const int n_my = split < n_tiles ? (n_tiles - split + p.n_splits - 1) / p.n_splits : 0;
  const bool final_out = p.n_splits == 1;
  const int halves_here = p.split_d ? 1 : Cfg::kHalves;            // halves of D this CTA accumulates
  const int d_first = p.split_d ? dz * Cfg::kOCols : 0;
  if (n_my == 0) {
    if (final_out) {
      // a row without keys (a padding row): zeros
      for (int i = tid; i < n_heads * (Cfg::kOCols * halves_here / 8); i += kTcThreads) {
        const int h = i / (Cfg::kOCols * halves_here / 8), c = i % (Cfg::kOCols * halves_here / 8);
        *reinterpret_cast<uint4*>(p.out + 1ll * r * p.ldo + 1ll * h * D + d_first + c * 8) = make_uint4(0, 0, 0, 0);
      }
    } else if (dz == 0 && tid < n_heads) {
      float* ml = p.part_ml + ((1ll * r * p.n_splits + split) * p.heads + tid) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&k_full[b], 4);
      mbar_init(&k_free[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4);
    }
    mbar_init(o_full, 1);
    mbar_init_fence();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (tid < p.rope_dim / 2) rope_cs_tc(pos, p.inv_freq[tid], &sCos[tid], &sSin[tid]);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- Q tile: RoPE on the tail, zero rows for the heads this rank does not have, UMMA-canonical layout
  {
    const int rope0 = D - p.rope_dim;
    const uint32_t sq = smem_u32(sQ);
    for (int idx = tid; idx < kTcHeads * CH; idx += kTcThreads) {
      const int h = idx / CH, ch = idx % CH;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (h < n_heads) {
        raw = *reinterpret_cast<const uint4*>(p.q + 1ll * r * p.ldq + p.q_off + 1ll * h * D + ch * 8);
        if (ch * 8 >= rope0) {
          __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
          for (int q2 = 0; q2 < 4; ++q2) {
            const float2 f = __bfloat1622float2(v[q2]);
            const int t = (ch * 8 + 2 * q2 - rope0) / 2;
            const float c = sCos[t], sn = sSin[t];
            v[q2] = __floats2bfloat162_rn(f.x * c - f.y * sn, f.y * c + f.x * sn);
          }
        }
      }
      st_shared16(sq + tile_off(h, ch), raw);
    }
  }
  fence_async_smem();
  __syncthreads();

  if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------ gather: 16 keys of every tile per warp
    const int lw = warp - 4;
    const long long row_bytes = p.kv_row_bytes > 0 ? p.kv_row_bytes : 2ll * D;
    const long long comp_bytes = p.comp_row_bytes > 0 ? p.comp_row_bytes : row_bytes;
    bool ok = true;
    for (int j = 0; j < n_my && ok; ++j) {
      const int tile = split + j * p.n_splits;
      const int b = j & 1;
      if (j >= 2) {
        ok = mbar_wait(&k_free[b], ((j >> 1) - 1) & 1, p.status, 400);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const int k0 = tile * kTcKeys + lw * 16;           // this warp's first key
      const uint8_t* my_ptr = nullptr;                   // lanes 0-15: address of key k0 + lane
      int my_fp4 = 0;
      if (lane < 16) {
        const int jk = k0 + lane;
        if (jk < n_keys) {
          if (jk < n_w) {
            const int kp = lo_pos + jk;
            my_ptr = p.win + (1ll * slot * p.ring + (kp % p.ring)) * row_bytes;
          } else {
            const int id = p.sel[1ll * r * p.k + (jk - n_w)];
            if (id >= 0) {
              const int page = p.page_table[1ll * slot * p.max_pages + id / p.page_rows];
              if (page >= 0) {
                my_ptr = p.comp_pool + (1ll * page * p.page_rows + id % p.page_rows) * comp_bytes;
                my_fp4 = p.comp_row_bytes > 0 ? 1 : 0;
              }
            }
          }
        }
      }
      const uint32_t kb = smem_u32(sK + b * Cfg::kTile);
      const uint32_t null_mask = __ballot_sync(0xffffffffu, my_ptr == nullptr) & 0xffffu;
      const uint32_t fp4_mask = __ballot_sync(0xffffffffu, my_fp4 != 0) & 0xffffu;
      if (p.kv_row_bytes == 0) {
        // bf16 rows: asynchronous 16-byte copies straight into the swizzled tile
#pragma unroll 4
        for (int kk = 0; kk < 16; ++kk) {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(
              __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_ptr), kk));
          const int key = lw * 16 + kk;
          if (src == nullptr) {
            for (int ch = lane; ch < CH; ch += 32) st_shared16(kb + tile_off(key, ch), make_uint4(0, 0, 0, 0));
          } else {
            for (int ch = lane; ch < CH; ch += 32) cp_async16(kb + tile_off(key, ch), src + ch * 16);
          }
        }
      } else {
        // quantised rows: every load of the warp's 16 keys is issued before the first conversion.
        //   FP8 row: D e4m3 values, then one UE8M0 scale per 32 values; lane u expands values [16u, 16u+16)
        //   FP4 row: D/2 bytes of e2m1 pairs, then one E4M3 scale per 16 values; lane u expands values [32u, 32u+32)
        uint4 raw[16];
        uint32_t scs[16];
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(
              __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_ptr), kk));
          const bool fp4 = (fp4_mask >> kk) & 1u;
          raw[kk] = make_uint4(0, 0, 0, 0);
          scs[kk] = 0;
          if (src != nullptr && lane < (fp4 ? D / 32 : D / 16)) {
            raw[kk] = __ldg(reinterpret_cast<const uint4*>(src + lane * 16));
            scs[kk] = fp4 ? static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(src + D / 2 + 2 * lane)))
                          : static_cast<uint32_t>(__ldg(src + D + (lane >> 1)));
          }
        }
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const int key = lw * 16 + kk;
          if ((null_mask >> kk) & 1u) {
            for (int ch = lane; ch < CH; ch += 32) st_shared16(kb + tile_off(key, ch), make_uint4(0, 0, 0, 0));
          } else if (!((fp4_mask >> kk) & 1u)) {
            if (lane < D / 16) {
              const float sc = __uint_as_float(scs[kk] << 23);            // exact: e4m3 value times a power of two
              const __nv_fp8x2_storage_t* q2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw[kk]);
              uint4 o[2];
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(q2[i], __NV_E4M3)));
                o2[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
              }
              st_shared16(kb + tile_off(key, 2 * lane), o[0]);
              st_shared16(kb + tile_off(key, 2 * lane + 1), o[1]);
            }
          } else if (lane < D / 32) {
            const uint32_t w4[4] = {raw[kk].x, raw[kk].y, raw[kk].z, raw[kk].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const __half_raw hs = __nv_cvt_fp8_to_halfraw(
                  static_cast<__nv_fp8_storage_t>((scs[kk] >> (8 * (c >> 1))) & 0xff), __NV_E4M3);
              const float sc = __half2float(__half(hs));                  // exact: 2-bit mantissa times 4-bit mantissa
              uint4 o;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                o2[i] = __floats2bfloat162_rn(e2m1_value((w4[c] >> (8 * i)) & 15u) * sc,
                                              e2m1_value((w4[c] >> (8 * i + 4)) & 15u) * sc);
              st_shared16(kb + tile_off(key, 4 * lane + c), o);
            }
          }
        }
      }
      cp_async_drain();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&k_full[b]);
    }
    cp_async_drain();
  } else if (warp == 8) {
    // ------------------------------------------------------------ MMA issue (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(kTcHeads, kTcKeys, 1u, 1u);
      constexpr uint32_t idesc_pv = umma_idesc_bmn(kTcHeads, Cfg::kOCols, 1u, 1u);
      const uint32_t sq = smem_u32(sQ), sk = smem_u32(sK), sp = smem_u32(sP);
      int next_s = 0, next_pv = 0;
      long long start = clock64();
      uint32_t spins = 0;
      while (next_pv < n_my) {
        bool progressed = false;
        if (next_s < n_my && next_s < next_pv + 2) {
          const int b = next_s & 1;
          if (mbar_try_wait(&k_full[b], (next_s >> 1) & 1)) {
            tc_fence_after();
            const uint32_t kt = sk + b * Cfg::kTile;
#pragma unroll 4
            for (int k = 0; k < D / 16; ++k) {
              const uint32_t off = (k >> 2) * kPanelBytes + (k & 3) * 32;
              umma_bf16(tmem_base + Cfg::kSCol + kTcKeys * b, umma_desc_sw128(sq + off), umma_desc_sw128(kt + off),
                        idesc_s, k > 0 ? 1u : 0u);
            }
            tc_commit(&s_full[b]);
            ++next_s;
            progressed = true;
          }
        }
        if (next_pv < next_s) {
          const int b = next_pv & 1;
          if (mbar_try_wait(&p_full[b], (next_pv >> 1) & 1)) {
            tc_fence_after();
            const uint32_t kt = sk + b * Cfg::kTile;
#pragma unroll
            for (int ks = 0; ks < kTcKeys / 16; ++ks) {
              const uint64_t adesc = umma_desc_sw128(sp + b * kPanelBytes + ks * 32);
              for (int h = 0; h < halves_here; ++h) {
                const int panel0 = (p.split_d ? dz : h) * (Cfg::kOCols / 64);
                const uint64_t bdesc = umma_desc_sw128_mn(kt + panel0 * kPanelBytes + ks * 2048, kPanelBytes, 1024);
                umma_bf16(tmem_base + (static_cast<uint32_t>(h * 16) << 16), adesc, bdesc, idesc_pv,
                          (next_pv > 0 || ks > 0) ? 1u : 0u);
              }
            }
            tc_commit(&k_free[b]);
            if (next_pv == n_my - 1) tc_commit(o_full);
            ++next_pv;
            progressed = true;
          }
        }
        if (progressed) {
          start = clock64();
          spins = 0;
        } else if ((++spins & 0x3ff) == 0) {
          if (clock64() - start > DS41_WAIT_LIMIT_CYCLES ||
              (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != kStatusOk)) {
            if (p.status != nullptr && atomicCAS(p.status, kStatusOk, kStatusMbarTimeout) == kStatusOk) {
              p.status[1] = 410;
              p.status[2] = static_cast<int>(blockIdx.y);
              p.status[3] = next_s * 1000 + next_pv;
            }
            break;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax, correction, epilogue (warps 0-3)
    const int hsel = lane & 15, half = lane >> 4;
    const int head = warp * 16 + hsel;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float scale2 = p.scale * kLog2e;
    const bool o_owner = half < halves_here;          // lanes 16-31 hold the second half of D when it is interleaved
    float m_ref = -INFINITY, l = 0.f;                 // per head (lanes 0-15), in log2 units
    bool ok = true;
    for (int j = 0; j < n_my && ok; ++j) {
      const int tile = split + j * p.n_splits;
      const int b = j & 1;
      const int k_cnt = min(kTcKeys, n_keys - tile * kTcKeys);
      ok = mbar_wait(&s_full[b], (j >> 1) & 1, p.status, 420);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(t_lane + Cfg::kSCol + kTcKeys * b, v0);
      tmem_ld_32x32(t_lane + Cfg::kSCol + kTcKeys * b + 32, v1);
      tmem_wait_ld();
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float a = c < k_cnt ? __uint_as_float(v0[c]) * scale2 : -INFINITY;
        const float bb = c + 32 < k_cnt ? __uint_as_float(v1[c]) * scale2 : -INFINITY;
        v0[c] = __float_as_uint(a);
        v1[c] = __float_as_uint(bb);
        mx = fmaxf(mx, fmaxf(a, bb));
      }
      const bool need = lane < 16 && mx > m_ref + kRescaleStep;
      if (__any_sync(0xffffffffu, need)) {
        // the reference of every head of this quadrant moves to its running maximum; O and l follow
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = m_ref == -INFINITY ? 0.f : ex2(m_ref - m_new);
        l *= alpha;
        m_ref = m_new;
        if (j > 0) {
          const float a_o = __shfl_sync(0xffffffffu, alpha, hsel);
          ok = mbar_wait(&k_free[(j - 1) & 1], ((j - 1) >> 1) & 1, p.status, 421);     // P V of the previous tile
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
      // P = 2^(s - reference) in bf16; the row sum adds the rounded values (what the tensor core multiplies)
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const __nv_bfloat162 e = __floats2bfloat162_rn(ex2(__uint_as_float(v0[c]) - m_ref),
                                                       ex2(__uint_as_float(v0[c + 1]) - m_ref));
        const __nv_bfloat162 f = __floats2bfloat162_rn(ex2(__uint_as_float(v1[c]) - m_ref),
                                                       ex2(__uint_as_float(v1[c + 1]) - m_ref));
        const float2 ef = __bfloat1622float2(e), ff = __bfloat1622float2(f);
        sum += (ef.x + ef.y) + (ff.x + ff.y);
        pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&e);
        pk[16 + (c >> 1)] = *reinterpret_cast<const uint32_t*>(&f);
      }
      l += sum;
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
    }
    if (ok) ok = mbar_wait(o_full, 0, p.status, 430);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const float l_h = __shfl_sync(0xffffffffu, l, hsel);
      const float m_h = __shfl_sync(0xffffffffu, m_ref, hsel);
      float f = 1.f;
      if (final_out) {
        const float sink2 = (head < n_heads ? __ldg(p.sink + head) : 0.f) * kLog2e;
        const float m_fin = fmaxf(m_h, sink2);
        const float w_o = ex2(m_h - m_fin);
        f = w_o / (l_h * w_o + ex2(sink2 - m_fin));
      } else if (lane < 16 && head < n_heads && dz == 0) {
        float* ml = p.part_ml + ((1ll * r * p.n_splits + split) * p.heads + head) * 2;
        ml[0] = m_h / kLog2e;
        ml[1] = l_h;
      }
      const int d_half0 = p.split_d ? dz * Cfg::kOCols : half * Cfg::kOCols;
      const int rope0 = D - p.rope_dim;
      const bool writer = o_owner && head < n_heads;
#pragma unroll 1
      for (int c0 = 0; c0 < Cfg::kOCols; c0 += 32) {
        uint32_t o[32];
        tmem_ld_32x32(t_lane + c0, o);
        tmem_wait_ld();
        const int d0 = d_half0 + c0;
        if (!writer) continue;
        if (final_out) {
          uint4 w[4];
          __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(w);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float a = __uint_as_float(o[c]) * f, bb = __uint_as_float(o[c + 1]) * f;
            const int t = d0 + c - rope0;
            if (t >= 0) {
              const float cs = sCos[t >> 1], sn = sSin[t >> 1];
              const float ra = a * cs + bb * sn, rb = bb * cs - a * sn;      // inverse rotation
              a = ra;
              bb = rb;
            }
            w2[c >> 1] = __floats2bfloat162_rn(a, bb);
          }
          uint4* dst = reinterpret_cast<uint4*>(p.out + 1ll * r * p.ldo + 1ll * head * D + d0);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = w[i];
        } else {
          float4* dst = reinterpret_cast<float4*>(p.part_o + ((1ll * r * p.n_splits + split) * p.heads + head) * D + d0);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                                 __uint_as_float(o[4 * i + 3]));
        }
      }
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
  dim3 grid(p.n_splits, p.rows, p.split_d ? Cfg::kHalves : 1);
  return launch_pdl(attend_tc_kernel<D>, grid, dim3(kTcThreads), Cfg::kSmem, stream, p);
}

}  // namespace ds41

using namespace ds41;

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
  p.split_d = (a->split_d != 0 && a->D == 512) ? 1 : 0;
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
