// Tensor-core GEMM for sm_100a:  D[m,n] = sum_k A[m,k] * B[n,k]   (both operands K-major)
//
// One persistent warp-specialised kernel: warp 0 streams A/B tiles with TMA into a multi-stage
// shared-memory ring, warp 1 issues tcgen05.mma into double-buffered TMEM accumulators, warps 2-5
// drain TMEM with tcgen05.ld and write the result.  Kinds: bf16, fp8 e4m3 (unscaled) and MX
// block-scaled fp8 (UE8M0 scale per 32 elements, scale factors copied into TMEM with tcgen05.cp).
// Split-K writes fp32 partial planes; "transposed" output serves the swap-AB decode orientation
// where the weight matrix is the M operand and the few token rows are the N operand.
//
// Capability parity: replaces the reference's AOT block-scaled dense GEMMs
// (native/include/ds41rt_v41_fp8.h:6-47) and its cuBLAS fallbacks (native/cuda/kernels/v41_attention_ops.cu:130-155).
#include <cuda.h>

#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"
#include "ds41_tma.h"

namespace ds41 {

#ifndef DS41_SKINNY_STAGES
#define DS41_SKINNY_STAGES 8
#endif

constexpr int kBM = 128;
constexpr int kTileKBytes = 128;       // one 128-byte swizzle span of K per stage
constexpr int kGemmThreads = 256;      // warps: 0 TMA, 1 MMA, 2-5 epilogue, 6-7 all-gather copiers
constexpr int kStagingBytes = 32768;   // TMA-store staging: 4 epilogue warps x 2 buffers x [32 rows][128 B]

// tensor maps of the TMA-store epilogue (mode 6): m[0] = the output, or with reduce-scatter m[d] = this rank's slot
// in rank d's buffer
struct StoreMaps {
  CUtensorMap m[8];
};

struct GemmParams {
  int M, N, K;            // K in elements
  int batch;
  int k_splits;
  int out_mode;           // 0 bf16 [m,n]; 1 f32 [m,n]; 2 bf16 [n,m]; 3 f32 [n,m];
                          // 4 (DUAL) bf16 [n,m] = swiglu(gate,up)*row_w; 5 f32 [n,m] where row_w != 0;
                          // 6 bf16 [m,n] staged in shared memory and written by TMA stores; 7 scatter rows;
                          // 8 indexer scores: rows of M are (query, head) pairs, 32 heads per query; out[query][n] =
                          //   sum_head relu(acc) * row_w[query][head], -inf at n >= col_limit[query]
  long long ldo;          // leading dimension of the output in elements
  long long out_batch_stride;
  long long out_split_stride;
  void* out;
  const uint8_t* sfa;     // MX kinds: scale-factor atoms of A / B
  const uint8_t* sfb;
  long long sfa_batch_stride;
  long long sfb_batch_stride;
  // grouped (MoE) extensions
  const int* batch_map;   // optional: A-operand batch coordinate of logical batch b
  const int* n_active;    // optional device scalar: only logical batches < *n_active run
  int b_batch_kind;       // B-operand batch coordinate: 0 = same as A, 1 = always 0, 2 = logical b
  int up_row_offset;      // DUAL: row offset of the second ("up") A tile (= intermediate size)
  const float* row_w;     // modes 4/5: per (logical batch, n) weight, [batch][row_w_ld]
  int row_w_ld;
  float act_limit;        // mode 4: SwiGLU clamp
  int static_operand;     // 1: A holds weights, 2: B holds weights (may be fetched before the dependency wait)
  float alpha;            // kind 3: product of the two tensors' global scales, applied to the accumulators
  const float* alpha_batch;   // optional extra factor per A batch (one global scale per expert)
  // completion signal folded into the kernel: the CTA that finishes last bumps *sig_epoch and stores it to sig_flags[..]
  unsigned int* sig_counter;
  unsigned int* sig_epoch;
  unsigned int* const* sig_flags;
  int sig_world;
  int a_fp4;              // MX kind: A holds e2m1 values (packed in global memory, one per byte in shared memory)
  // grouped tokens (expert-parallel prefill, swap-AB): the N operand is a flat buffer of rows sorted by expert;
  // tile j covers rows [tile_row0[j], tile_end[j]) of expert tile_group[j]; *n_tiles_dev tiles are live
  const int* tile_group;
  const int* tile_row0;
  const int* tile_end;
  const int* n_tiles_dev;
  // generic dependency on peers (bounded wait by the producer before its first dependent load)
  const uint32_t* const* wait_flags;
  const uint32_t* wait_epoch;
  int wait_world;
  // mode 7: scatter rows to their source ranks (expert-parallel combine): meta[n] = {source rank, slot}
  const int2* scatter_meta;
  void* scatter_out[8];
  const int* col_limit;   // mode 8: visible keys per query row
  // fused collectives over peer memory (normal orientation: A = activations, rows sharded by rank)
  // all-gather -> GEMM (push model): A is this rank's copy of the gathered matrix; rows [r*ag_rows, (r+1)*ag_rows)
  // belong to rank r.  The copier warps push this rank's rows into every peer's copy (ag_bufs[d]) in
  // (128-row tile, K chunk) units and add 1 to the peer's arrival counter [src][tile] per unit; the TMA producer
  // waits until a remote tile's counter reaches epoch * ag_chunks before loading it from local memory.
  int ag_world, ag_rank, ag_rows, ag_chunks;
  long long a_row_bytes;                  // bytes between rows of A
  void* ag_bufs[8];
  uint32_t* ag_arrive[8];                 // counters [ag_world][ag_rows / 128] on every rank
  const uint32_t* ag_epoch;
  int rs_world, rs_rank, rs_rows;         // GEMM -> reduce-scatter: output rows of rank d go to rank d (mode 6 maps
  void* rs_out[8];                        // or, modes 0/1, rs_out[d] slot rs_rank)
  int* status;
};

template <int BN, int KIND, int DUAL = 0>
struct GemmCfg {
  static constexpr int kElemBytes = (KIND == 0) ? 2 : 1;
  // elements of K per stage: one 128-byte swizzle span (kind 3 packs two e2m1 values per byte)
  static constexpr int kBK = (KIND == 3) ? 2 * kTileKBytes : kTileKBytes / kElemBytes;
  static constexpr int kSfPerTile = (KIND == 3) ? 4 : 1;               // 512-byte scale atoms per 128 rows per stage
  static constexpr bool kScaled = (KIND == 2 || KIND == 3);
  static constexpr int kATile = kBM * kTileKBytes;                     // 16 KiB
  static constexpr int kABytes = kATile * (DUAL ? 2 : 1);
  static constexpr int kBBytes = BN * kTileKBytes;
  static constexpr int kTilesA = DUAL ? 2 : 1;
  static constexpr int kTilesB = (BN + 127) / 128;
  static constexpr int kAtomsA = kTilesA * kSfPerTile;
  static constexpr int kAtomsB = kTilesB * kSfPerTile;
  // scale-factor atoms (512 B each), padded so every stage keeps its 1024-byte tile alignment
  static constexpr int kSfBytes = kScaled ? ((512 * (kAtomsA + kAtomsB) + 1023) / 1024 * 1024) : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;
  static constexpr int kStaging = (!DUAL && BN >= 64) ? kStagingBytes : 0;
  static constexpr int kStagesRaw = ((kStaging ? 194 : 200) * 1024) / kStageBytes;
  // Skinny decode tiles (BN <= 32) keep the ring short enough for two CTAs of consecutive launches to share an SM: the
  // next kernel's set-up and its weight prefetch then overlap the tail of the previous one (programmatic launch).
  static constexpr int kStageCap = (BN <= 32) ? DS41_SKINNY_STAGES : 8;
  static constexpr int kStages = kStagesRaw > kStageCap ? kStageCap : kStagesRaw;
  static constexpr int kSfCols = kScaled ? 4 * (kAtomsA + kAtomsB) : 0;               // TMEM columns per stage
  static constexpr int kAccCols = (BN < 32 ? 32 : BN) * (DUAL ? 2 : 1);
  // Two accumulator sets let the epilogue of one tile overlap the MMAs of the next.  The widest block-scaled dual tile
  // (128 tokens x gate + up) leaves room for only one beside its scale columns; it is still the better trade there:
  // each weight byte fetched from L2 serves twice the tokens of a 64-wide tile.
  static constexpr int kAccStages = (2 * kAccCols + kStages * kSfCols <= 512) ? 2 : 1;
  static constexpr int kTmemNeeded = kAccStages * kAccCols + kStages * kSfCols;
  static constexpr int kTmemCols = kTmemNeeded <= 32 ? 32 : kTmemNeeded <= 64 ? 64 : kTmemNeeded <= 128 ? 128
                                   : kTmemNeeded <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStaging + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(kTmemNeeded <= 512, "TMEM budget exceeded");
  static_assert(kStages >= 2, "not enough shared memory for two stages");
};

// Tile order: bands of kBandTiles m-tiles; inside a band the m-tile runs fastest, then the n-tile.  The CTAs of one
// wave then share a few n-tiles of B and a band of A that stays in L2 while the band sweeps N, instead of streaming all
// of A from DRAM once per n-tile.  Returns the remaining (split, batch) index.
constexpr int kBandTiles = 16;
__device__ __forceinline__ long long decode_tile(long long t, int m_tiles, int n_tiles, int band_tiles, int& mt,
                                                 int& nt) {
  const long long per_mn = 1ll * m_tiles * n_tiles;
  const long long outer = t / per_mn;
  const int r = static_cast<int>(t - outer * per_mn);
  const int per_band = band_tiles * n_tiles;
  const int band = r / per_band;
  const int rb = r - band * per_band;
  const int band_rows = min(band_tiles, m_tiles - band * band_tiles);
  nt = rb / band_rows;
  mt = band * band_tiles + (rb - nt * band_rows);
  return outer;
}

template <int BN, int KIND, int DUAL>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ StoreMaps stm, GemmParams p) {
  using Cfg = GemmCfg<BN, KIND, DUAL>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* staging = smem + S * Cfg::kStageBytes;
  uint8_t* bar_base = staging + Cfg::kStaging;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty = full + S;
  uint64_t* acc_full = empty + S;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* epi_bar = acc_empty + 2;        // the four epilogue warps meet here when they share a staging buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles = (p.M + kBM - 1) / kBM;
  const bool table = p.tile_group != nullptr;
  if (table) pdl_wait();              // the tile table is produced by an earlier kernel
  const int n_tiles = table ? *p.n_tiles_dev : (p.N + BN - 1) / BN;
  // grouped experts sweep all weight tiles of an expert per token tile; dense GEMMs use bands
  const int band_tiles = table ? m_tiles : kBandTiles;
  const int kb_total = (p.K + Cfg::kBK - 1) / Cfg::kBK;
  const int kb_per_split = (kb_total + p.k_splits - 1) / p.k_splits;
  pdl_launch_dependents();
  int batch_run = table ? 1 : p.batch;
  if (p.n_active != nullptr) {
    pdl_wait();                       // the active-expert count is produced by an earlier kernel
    batch_run = min(batch_run, *p.n_active);
  }
  const long long tiles = 1ll * m_tiles * n_tiles * p.k_splits * batch_run;
  // with a fused collective every rank starts on its own rows and walks the peers in ring order
  // reduce-scatter: the rows of the next rank first (their stores travel while the rest computes), the own rows last
  const int rot = p.ag_world > 0 ? p.ag_rank * (p.ag_rows / kBM)
                  : (p.rs_world > 0 ? ((p.rs_rank + 1) % p.rs_world) * (p.rs_rows / kBM) : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_init(epi_bar, 4);
    mbar_init_fence();
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // 4-bit A tiles occupy one byte per element in shared memory but the copy engine accounts the packed bytes
    const uint32_t kStageTx = (p.a_fp4 ? Cfg::kABytes / 2 : Cfg::kABytes) + Cfg::kBBytes +
                              (Cfg::kScaled ? 512 * (Cfg::kAtomsA + Cfg::kAtomsB) : 0);
    // Weight tiles of the first stages do not depend on the previous kernel: fetch them before waiting for it.
    int prefetched = 0;
    if (p.static_operand != 0 && p.n_active == nullptr && p.batch_map == nullptr && !table && blockIdx.x < tiles) {
      long long r = blockIdx.x;
      int mt, nt;
      r = decode_tile(r, m_tiles, n_tiles, band_tiles, mt, nt);
      const int sp = static_cast<int>(r % p.k_splits); r /= p.k_splits;
      const int b = static_cast<int>(r);
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(kb_total, kb0 + kb_per_split);
      prefetched = min(S, kb1 - kb0);
      for (int i = 0; i < prefetched; ++i) {
        uint8_t* sa = smem + i * Cfg::kStageBytes;
        mbar_expect_tx(&full[i], kStageTx);
        if (p.static_operand == 1) {
          tma_load_3d(sa, &tmA, &full[i], (kb0 + i) * Cfg::kBK, mt * kBM, b);
          if constexpr (DUAL)
            tma_load_3d(sa + Cfg::kATile, &tmA, &full[i], (kb0 + i) * Cfg::kBK, p.up_row_offset + mt * kBM, b);
        } else {
          tma_load_3d(sa + Cfg::kABytes, &tmB, &full[i], (kb0 + i) * Cfg::kBK, nt * BN, p.b_batch_kind == 1 ? 0 : b);
        }
      }
    }
    pdl_wait();
    if (p.wait_flags != nullptr && p.wait_world > 1) {
      for (int k = 0; k < p.wait_world && ok; ++k)
        if (!flag_wait_ge(p.wait_flags[k], *p.wait_epoch, p.status, 120 + k)) ok = false;
    }
    for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
      long long r = t;
      int mt, nt;
      r = decode_tile(r, m_tiles, n_tiles, band_tiles, mt, nt);
      const int sp = static_cast<int>(r % p.k_splits); r /= p.k_splits;
      const int b = table ? p.tile_group[nt] : static_cast<int>(r);
      const int n_base = table ? p.tile_row0[nt] : nt * BN;
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(kb_total, kb0 + kb_per_split);
      const int mt_eff = rot ? (mt + rot) % m_tiles : mt;
      const int a_row = mt_eff * kBM;
      if (p.ag_world > 1) {
        const int src = a_row / p.ag_rows;
        if (src != p.ag_rank) {
          // the rows were pushed by rank src's copier warps: wait for all K chunks of this 128-row tile
          const int j = (a_row - src * p.ag_rows) / kBM;
          const uint32_t need = *p.ag_epoch * static_cast<uint32_t>(p.ag_chunks);
          if (!flag_wait_ge(p.ag_arrive[p.ag_rank] + src * (p.ag_rows / kBM) + j, need, p.status, 110 + src)) {
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
      }
      for (int kb = kb0; kb < kb1; ++kb) {
        const bool early = prefetched > 0;      // this stage's barrier is armed and its weight tile is in flight
        if (early) --prefetched;
        if (!early && !mbar_wait(&empty[stage], phase ^ 1, p.status, 100)) { ok = false; break; }
        uint8_t* sa = smem + stage * Cfg::kStageBytes;
        uint8_t* sb = sa + Cfg::kABytes;
        if (!early) mbar_expect_tx(&full[stage], kStageTx);
        const int ba = p.batch_map != nullptr ? p.batch_map[b] : b;
        const int bb = p.b_batch_kind == 0 ? ba : (p.b_batch_kind == 1 ? 0 : b);
        if (!early || p.static_operand != 1) {
          tma_load_3d(sa, &tmA, &full[stage], kb * Cfg::kBK, a_row, ba);
          if constexpr (DUAL)
            tma_load_3d(sa + Cfg::kATile, &tmA, &full[stage], kb * Cfg::kBK, p.up_row_offset + mt * kBM, ba);
        }
        if (!early || p.static_operand != 2) tma_load_3d(sb, &tmB, &full[stage], kb * Cfg::kBK, n_base, bb);
        if constexpr (Cfg::kScaled) {
          // scale-factor atoms: [row_atom][k_atom][512 B]; kSfPerTile consecutive k_atoms per stage and 128 rows
          // (MX: one atom = 128 K elements with a UE8M0 scale per 32; NVFP4: four atoms of 64 K elements, E4M3 per 16)
          constexpr int kSf = Cfg::kSfPerTile;
          uint8_t* ssf = sb + Cfg::kBBytes;
          const long long ka = 1ll * kb * kSf;
          const long long n_ka = 1ll * kb_total * kSf;
          bulk_load(ssf, p.sfa + ba * p.sfa_batch_stride + (1ll * mt * n_ka + ka) * 512, 512 * kSf, &full[stage]);
          if constexpr (DUAL) {
            const long long mt_up = p.up_row_offset / 128 + mt;
            bulk_load(ssf + 512 * kSf, p.sfa + ba * p.sfa_batch_stride + (mt_up * n_ka + ka) * 512, 512 * kSf, &full[stage]);
          }
#pragma unroll
          for (int a = 0; a < Cfg::kTilesB; ++a) {
            const long long ra = n_base / 128 + a;
            bulk_load(ssf + 512 * (Cfg::kAtomsA + a * kSf), p.sfb + bb * p.sfb_batch_stride + (ra * n_ka + ka) * 512,
                      512 * kSf, &full[stage]);
          }
        }
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop with uniform control flow; `leader` predicates the tensor-core instructions
    // themselves.  Issued from inside a one-lane branch, every instruction's descriptors took a detour through the
    // divergent path that cost more than a K = 32 FP8 instruction takes to execute (tensor pipe 30 % busy in the
    // block-scaled expert GEMMs).
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr uint32_t kFmt = (KIND == 0) ? 1u : 0u;   // bf16 / e4m3
    for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
      int mt_unused, nt;
      const long long r = decode_tile(t, m_tiles, n_tiles, band_tiles, mt_unused, nt);
      const int sp = static_cast<int>(r % p.k_splits);
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(kb_total, kb0 + kb_per_split);
      ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.status, 200);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * Cfg::kAccCols;
      // A tile of the expert table that holds fewer than BN token rows multiplies only as many columns as it has
      // (rounded up to the instruction's granularity of 16): the last tile of an expert is mostly padding otherwise.
      uint32_t n_mma = BN;
      if (table) {
        const int valid = p.tile_end[nt] - p.tile_row0[nt];
        if (valid < BN) n_mma = static_cast<uint32_t>(max(16, (valid + 15) & ~15));
      }
      [[maybe_unused]] const uint32_t idesc_t = umma_idesc(kBM, n_mma, kFmt, kFmt);
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = mbar_wait(&full[stage], phase, p.status, 201);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
        const uint32_t sb = sa + Cfg::kABytes;
        const uint64_t adesc = umma_desc_sw128(sa);
        const uint64_t bdesc = umma_desc_sw128(sb);
        if constexpr (Cfg::kScaled) {
          const uint32_t ssf = sb + Cfg::kBBytes;
          const uint32_t sf_t = tmem_base + Cfg::kAccStages * Cfg::kAccCols + stage * Cfg::kSfCols;
#pragma unroll
          for (int a = 0; a < Cfg::kAtomsA + Cfg::kAtomsB; ++a)
            tmem_cp_32x128b_warpx4_if(leader, sf_t + 4 * a, umma_desc_plain(ssf + 512 * a, 16, 128));
          // B scale columns: rows of this n-tile start (nt*BN % 128)/32 columns into the atom
          const uint32_t n_base_u = table ? static_cast<uint32_t>(p.tile_row0[nt]) : static_cast<uint32_t>(nt) * BN;
          const uint32_t sfb_t = sf_t + 4 * Cfg::kAtomsA + (n_base_u & 127u) / 32u;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            if constexpr (KIND == 2) {
              // one atom per stage; instruction k uses byte k of every 32-bit scale cell
              const uint32_t id = umma_idesc_bs(kBM, n_mma, p.a_fp4 ? 5u : 0u, 0, 1, k, k);   // e2m1 = 5, e4m3 = 0
              umma_mxf8_if(leader, d_tmem, adesc + 2 * k, bdesc + 2 * k, id, accum, sf_t, sfb_t);
              if constexpr (DUAL) {
                const uint64_t adesc2 = umma_desc_sw128(sa + Cfg::kATile);
                umma_mxf8_if(leader, d_tmem + Cfg::kAccCols / 2, adesc2 + 2 * k, bdesc + 2 * k, id, accum, sf_t + 4, sfb_t);
              }
            } else {
              // NVFP4: instruction k (64 K elements) uses atom k: four E4M3 scales per row fill one 32-bit cell
              const uint32_t id = umma_idesc_bs(kBM, n_mma, 1u, 1u, 0, 0, 0);                // e2m1 x e2m1, UE4M3 scales
              umma_nvf4_if(leader, d_tmem, adesc + 2 * k, bdesc + 2 * k, id, accum, sf_t + 4 * k, sfb_t + 4 * k);
              if constexpr (DUAL) {
                const uint64_t adesc2 = umma_desc_sw128(sa + Cfg::kATile);
                umma_nvf4_if(leader, d_tmem + Cfg::kAccCols / 2, adesc2 + 2 * k, bdesc + 2 * k, id, accum, sf_t + 16 + 4 * k,
                          sfb_t + 4 * k);
              }
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < kTileKBytes / 32; ++k) {
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            if constexpr (KIND == 0) umma_bf16_if(leader, d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_t, accum);
            else umma_f8_if(leader, d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_t, accum);
            if constexpr (DUAL) {
              const uint64_t adesc2 = umma_desc_sw128(sa + Cfg::kATile);
              if constexpr (KIND == 0) umma_bf16_if(leader, d_tmem + Cfg::kAccCols / 2, adesc2 + 2 * k, bdesc + 2 * k, idesc_t, accum);
              else umma_f8_if(leader, d_tmem + Cfg::kAccCols / 2, adesc2 + 2 * k, bdesc + 2 * k, idesc_t, accum);
            }
          }
        }
        tc_commit_if(leader, &empty[stage]);       // frees the smem stage when these MMAs retire
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
      tc_commit_if(leader && ok, &acc_full[acc]);
      acc = (acc + 1 == Cfg::kAccStages) ? 0 : acc + 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t st_pair = 0;                      // mode 6: staging buffer parity of this warp
    uint32_t epi_count = 0;                    // mode 7: chunks staged so far (buffer = count & 1, barrier phase)
    for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
      long long r = t;
      int mt, nt;
      r = decode_tile(r, m_tiles, n_tiles, band_tiles, mt, nt);
      const int sp = static_cast<int>(r % p.k_splits); r /= p.k_splits;
      const int b = table ? p.tile_group[nt] : static_cast<int>(r);
      const int n_base = table ? p.tile_row0[nt] : nt * BN;
      const int n_lim = table ? p.tile_end[nt] : p.N;
      // per-column metadata (route weight / return address) of the first chunk, fetched while the MMAs still run;
      // every chunk then fetches the next chunk's before it starts its own stores
      constexpr int kChunkPre = BN >= 32 ? 32 : BN;
      const float* rw_base = (p.out_mode == 4 || p.out_mode == 5) ? p.row_w + (table ? 0ll : 1ll * b * p.row_w_ld) : nullptr;
      float rw_next = 0.f;
      int2 meta_next = make_int2(-1, -1);
      if (lane < kChunkPre && n_base + lane < n_lim) {
        if (rw_base != nullptr) rw_next = __ldcg(rw_base + n_base + lane);
        if (p.out_mode == 7) meta_next = __ldcg(p.scatter_meta + n_base + lane);
      }
      if (!mbar_wait(&acc_full[acc], acc_phase, p.status, 300)) { ok = false; break; }
      tc_fence_after();
      const int m = (rot ? (mt + rot) % m_tiles : mt) * kBM + quad * 32 + lane;
      // reduce-scatter: rows owned by rank d are stored into d's buffer, in the slot of this (source) rank
      char* rs_base = nullptr;
      long long rs_row = 0;
      if (p.rs_world > 0) {
        const int dst = m / p.rs_rows;
        rs_base = static_cast<char*>(p.rs_out[dst < p.rs_world ? dst : 0]);
        rs_row = 1ll * p.rs_rank * p.rs_rows + (m - dst * p.rs_rows);
      }
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * Cfg::kAccCols;
      const long long obase = (table ? 0ll : b * p.out_batch_stride) + sp * p.out_split_stride;
      constexpr int kChunk = BN >= 32 ? 32 : BN;
      float alpha = p.alpha;
      if (KIND == 3 && p.alpha_batch != nullptr) alpha *= __ldg(p.alpha_batch + (p.batch_map != nullptr ? p.batch_map[b] : b));
      // columns the tensor cores wrote for this tile (see n_mma in the issuer), in whole chunks
      const int n_cols = (table && p.out_mode != 6) ? min(BN, (max(n_lim - n_base, 0) + kChunk - 1) / kChunk * kChunk) : BN;
#pragma unroll 1
      for (int c = 0; c < n_cols; c += kChunk) {
        uint32_t v[32];
        if constexpr (kChunk == 32) {
          tmem_ld_32x32(t_row + c, v);
        } else if constexpr (kChunk == 16) {
          uint32_t v16[16];
          tmem_ld_32x16(t_row + c, v16);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = v16[j];
        } else {
          uint32_t v8[8];
          tmem_ld_32x8(t_row + c, v8);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = v8[j];
        }
        tmem_wait_ld();
        if constexpr (KIND == 3) {
#pragma unroll
          for (int j = 0; j < kChunk; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
        }
        const int n0 = n_base + c;
        const float rw_lane = rw_next;
        const int2 meta_lane = meta_next;
        rw_next = 0.f;
        meta_next = make_int2(-1, -1);
        if (c + kChunk < BN && lane < kChunk && n0 + kChunk + lane < n_lim) {
          if (rw_base != nullptr) rw_next = __ldcg(rw_base + n0 + kChunk + lane);
          if (p.out_mode == 7) meta_next = __ldcg(p.scatter_meta + n0 + kChunk + lane);
        }
        if (p.out_mode == 0) {
          if (m < p.M) {
            __nv_bfloat16* o = rs_base != nullptr ? reinterpret_cast<__nv_bfloat16*>(rs_base) + rs_row * p.ldo + n0
                                                  : reinterpret_cast<__nv_bfloat16*>(p.out) + obase + 1ll * m * p.ldo + n0;
            if (n0 + kChunk <= n_lim && (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < kChunk; j += 8) {
                uint4 q;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                q.x = *reinterpret_cast<uint32_t*>(&h0);
                q.y = *reinterpret_cast<uint32_t*>(&h1);
                q.z = *reinterpret_cast<uint32_t*>(&h2);
                q.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(o + j) = q;
              }
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (n0 + j < n_lim) o[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
            }
          }
        } else if (p.out_mode == 1) {
          if (m < p.M) {
            float* o = rs_base != nullptr ? reinterpret_cast<float*>(rs_base) + rs_row * p.ldo + n0
                                          : reinterpret_cast<float*>(p.out) + obase + 1ll * m * p.ldo + n0;
            if (n0 + kChunk <= n_lim && (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < kChunk; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (n0 + j < n_lim) o[j] = __uint_as_float(v[j]);
            }
          }
        } else if (p.out_mode == 2) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + obase + m;
          if (m < p.M) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              if (n0 + j < n_lim) o[1ll * (n0 + j) * p.ldo] = __float2bfloat16_rn(__uint_as_float(v[j]));
          }
        } else if (p.out_mode == 3) {
          float* o = reinterpret_cast<float*>(p.out) + obase + m;
          if (m < p.M) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              if (n0 + j < n_lim) o[1ll * (n0 + j) * p.ldo] = __uint_as_float(v[j]);
          }
        } else if (p.out_mode == 4) {
          if constexpr (DUAL) {
            // v = gate chunk; fetch the matching up chunk from the second accumulator half
            uint32_t u[32];
            if constexpr (kChunk == 32) {
              tmem_ld_32x32(t_row + Cfg::kAccCols / 2 + c, u);
            } else {
              uint32_t u16[16];
              tmem_ld_32x16(t_row + Cfg::kAccCols / 2 + c, u16);
#pragma unroll
              for (int j = 0; j < 16; ++j) u[j] = u16[j];
            }
            tmem_wait_ld();
            if constexpr (KIND == 3) {
#pragma unroll
              for (int j = 0; j < kChunk; ++j) u[j] = __float_as_uint(__uint_as_float(u[j]) * alpha);
            }
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + obase + m;
            // the chunk's route weights were fetched with one coalesced load and are handed out by shuffle: a load per
            // column would be ordered behind the previous column's store
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const float rwj = __shfl_sync(0xffffffffu, rw_lane, j);
              if (m < p.M && n0 + j < n_lim) {
                const float gte = fminf(bf16_round(__uint_as_float(v[j])), p.act_limit);
                const float upv = fminf(fmaxf(bf16_round(__uint_as_float(u[j])), -p.act_limit), p.act_limit);
                const float act = gte / (1.0f + __expf(-gte)) * upv * rwj;
                o[1ll * (n0 + j) * p.ldo] = __float2bfloat16_rn(act);
              }
            }
          }
        } else if (p.out_mode == 6) {
          if constexpr (Cfg::kStaging > 0) {
            // 64 columns (two chunks) per staging buffer: [32 rows][128 B] in the 128-byte swizzle, then one TMA store
            uint8_t* buf = staging + quad * 8192 + (st_pair & 1u) * 4096;
            const int half = (c >> 5) & 1;
            if (half == 0) {
              if (lane == 0) bulk_wait_group_read<1>();     // the store issued from this buffer two pairs ago has read it
              __syncwarp();
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1]));
              __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
              __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
              w.x = *reinterpret_cast<uint32_t*>(&h0);
              w.y = *reinterpret_cast<uint32_t*>(&h1);
              w.z = *reinterpret_cast<uint32_t*>(&h2);
              w.w = *reinterpret_cast<uint32_t*>(&h3);
              const int chunk16 = half * 4 + q;
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk16 ^ (lane & 7)) << 4)) = w;
            }
            if (half == 1) {
              fence_async_smem();
              __syncwarp();
              if (lane == 0) {
                const int m_tile0 = (rot ? (mt + rot) % m_tiles : mt) * kBM;
                int row0 = m_tile0 + quad * 32, z = b;
                const CUtensorMap* map = &stm.m[0];
                if (p.rs_world > 0) {
                  const int dst = m_tile0 / p.rs_rows;
                  map = &stm.m[dst];
                  row0 -= dst * p.rs_rows;
                  z = 0;
                }
                tma_store_3d(map, buf, n0 - 32, row0, z);
                bulk_commit_group();
              }
              ++st_pair;
            }
          }
        } else if (p.out_mode == 8) {
          // One epilogue warp = the 32 heads of one query row.  relu x head weight, then a butterfly that leaves the
          // sum over heads of column l on lane l (31 shuffles for 32 columns), then one coalesced row store.
          if constexpr (kChunk == 32) {
            const int qrow = m >> 5;
            const float wgt = m < p.M ? __ldg(p.row_w + 1ll * qrow * p.row_w_ld + lane) : 0.f;
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = fmaxf(__uint_as_float(v[j]), 0.f) * wgt;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
              const bool upper = (lane & off) != 0;
#pragma unroll
              for (int i = 0; i < off; ++i) {
                const float send = upper ? f[i] : f[i + off];
                const float keep = upper ? f[i + off] : f[i];
                f[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
              }
            }
            if (m < p.M && n0 + lane < n_lim) {
              const int lim = p.col_limit != nullptr ? __ldg(p.col_limit + qrow) : n_lim;
              reinterpret_cast<float*>(p.out)[obase + 1ll * qrow * p.ldo + n0 + lane] = n0 + lane < lim ? f[0] : -INFINITY;
            }
          }
        } else if (p.out_mode == 7) {
          // expert-parallel combine: column n is a received token row; its result row goes back to the rank it
          // came from, into that rank's combine buffer at the (token, route) slot - P2P stores from the epilogue.
          if constexpr (Cfg::kStaging > 0) {
            // The four warps transpose the chunk through shared memory ([32 tokens][128 features] bf16) so that half a
            // warp writes 256 contiguous bytes of one token: 8x fewer and 4x longer stores than one column per warp.
            uint8_t* buf = staging + (epi_count & 1u) * 8192;
            __nv_bfloat16* col = reinterpret_cast<__nv_bfloat16*>(buf) + quad * 32 + lane;
#pragma unroll
            for (int j = 0; j < kChunk; ++j) col[j * 128] = __float2bfloat16_rn(__uint_as_float(v[j]));
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_bar);
            if (!mbar_wait(epi_bar, epi_count & 1u, p.status, 310)) { ok = false; break; }
            ++epi_count;
            const int e = quad * 32 + lane;
            const int m_tile0 = (rot ? (mt + rot) % m_tiles : mt) * kBM;
            const int piece = e & 15;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int j = it * 8 + (e >> 4);
              const int src = __shfl_sync(0xffffffffu, meta_lane.x, j & 31);
              const int slot = __shfl_sync(0xffffffffu, meta_lane.y, j & 31);
              const int mm = m_tile0 + piece * 8;
              if (src >= 0 && src < 8 && slot >= 0 && mm < p.M) {
                const uint4 w = *reinterpret_cast<const uint4*>(buf + j * 256 + piece * 16);
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.scatter_out[src]) + 1ll * slot * p.ldo + mm;
                if (mm + 8 <= p.M) {
                  *reinterpret_cast<uint4*>(o) = w;
                } else {
                  const __nv_bfloat16* wh = reinterpret_cast<const __nv_bfloat16*>(&w);
                  for (int q = 0; q < 8 && mm + q < p.M; ++q) o[q] = wh[q];
                }
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int src = __shfl_sync(0xffffffffu, meta_lane.x, j);
              const int slot = __shfl_sync(0xffffffffu, meta_lane.y, j);
              if (m < p.M && src >= 0 && src < 8 && slot >= 0) {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.scatter_out[src]) + 1ll * slot * p.ldo + m;
                *o = __float2bfloat16_rn(__uint_as_float(v[j]));
              }
            }
          }
        } else {
          float* o = reinterpret_cast<float*>(p.out) + obase + m;
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const float rwj = __shfl_sync(0xffffffffu, rw_lane, j);
            if (m < p.M && rwj != 0.f) o[1ll * (n0 + j) * p.ldo] = __uint_as_float(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      acc = (acc + 1 == Cfg::kAccStages) ? 0 : acc + 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (p.out_mode == 6 && lane == 0) bulk_wait_group<0>();   // every TMA store of this warp has been performed
  } else if (warp >= 6) {
    // ------------------------------------------------------------ all-gather copiers (2 warps)
    if (p.ag_world > 1) {
      pdl_wait();
      const int ct = static_cast<int>(threadIdx.x) - 192;
      const int mt_shard = p.ag_rows / kBM;
      const int peers = p.ag_world - 1;
      const int units = mt_shard * peers * p.ag_chunks;
      const int chunk_bytes = static_cast<int>(1ll * p.K * Cfg::kElemBytes / p.ag_chunks);
      const int vec_row = chunk_bytes >> 4;
      const int total = kBM * vec_row;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int j = u % mt_shard;
        const int rr = u / mt_shard;
        const int d = (p.ag_rank + 1 + rr % peers) % p.ag_world;
        const int c = rr / peers;
        const long long off = (1ll * p.ag_rank * p.ag_rows + 1ll * j * kBM) * p.a_row_bytes + 1ll * c * chunk_bytes;
        const char* src = static_cast<const char*>(p.ag_bufs[p.ag_rank]) + off;
        char* dst = static_cast<char*>(p.ag_bufs[d]) + off;
        for (int i0 = 0; i0 < total; i0 += 64 * 8) {
          uint4 w[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * 64 + ct;
            if (i < total) w[q] = *reinterpret_cast<const uint4*>(src + (i / vec_row) * p.a_row_bytes + ((i % vec_row) << 4));
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * 64 + ct;
            if (i < total) *reinterpret_cast<uint4*>(dst + (i / vec_row) * p.a_row_bytes + ((i % vec_row) << 4)) = w[q];
          }
        }
        __threadfence_system();
        named_barrier(1, 64);
        if (ct == 0) flag_add_release(p.ag_arrive[d] + p.ag_rank * mt_shard + j, 1u);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  if (p.sig_counter != nullptr) __threadfence();          // this CTA's output stores, before it is counted as done
  __syncthreads();
  if (p.sig_counter != nullptr && warp == 0) {
    unsigned int last = 0;
    if (lane == 0) last = atomicAdd(p.sig_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
    last = __shfl_sync(0xffffffffu, last, 0);
    __syncwarp();                              // the other lanes order themselves after lane 0's view of the counter
    if (last) {
      __threadfence();
      uint32_t e = 0;
      if (lane == 0) {
        e = *p.sig_epoch + 1;
        *p.sig_epoch = e;
        *p.sig_counter = 0u;
      }
      e = __shfl_sync(0xffffffffu, e, 0);
      if (lane < p.sig_world) flag_store_release(const_cast<uint32_t*>(p.sig_flags[lane]), e);   // release at system scope
    }
  }
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != kStatusOk) {
    // A wait gave up: let copies that may still be in flight land before the CTA's memory goes away.
    const long long start = clock64();
    while (clock64() - start < 2000000ll) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int BN, int KIND, int DUAL = 0>
static cudaError_t launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& peer,
                               const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, KIND, DUAL>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, KIND, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(gemm_tc_kernel<BN, KIND, DUAL>, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, tmA, tmB, peer, p);
}

template <int KIND>
static cudaError_t dispatch_bn(int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const StoreMaps& peer,
                               const GemmParams& p, int grid, cudaStream_t stream) {
  if (p.out_mode == 4) {
    switch (bn) {
      case 16: return launch_gemm<16, KIND, 1>(tmA, tmB, peer, p, grid, stream);
      case 32: return launch_gemm<32, KIND, 1>(tmA, tmB, peer, p, grid, stream);
      case 64: return launch_gemm<64, KIND, 1>(tmA, tmB, peer, p, grid, stream);
      case 128:
        if constexpr (KIND < 3) return launch_gemm<128, KIND, 1>(tmA, tmB, peer, p, grid, stream);
        return cudaErrorInvalidValue;
      case 192:      // expert tiles of the block-scaled FP8 kind: one tile holds a whole expert of a typical pass
        if constexpr (KIND == 2) return launch_gemm<192, KIND, 1>(tmA, tmB, peer, p, grid, stream);
        return cudaErrorInvalidValue;
      default: return cudaErrorInvalidValue;
    }
  }
  switch (bn) {
    case 16: return launch_gemm<16, KIND>(tmA, tmB, peer, p, grid, stream);
    case 32: return launch_gemm<32, KIND>(tmA, tmB, peer, p, grid, stream);
    case 64: return launch_gemm<64, KIND>(tmA, tmB, peer, p, grid, stream);
    case 128: return launch_gemm<128, KIND>(tmA, tmB, peer, p, grid, stream);
    case 192:
      if constexpr (KIND == 2) return launch_gemm<192, KIND>(tmA, tmB, peer, p, grid, stream);
      return cudaErrorInvalidValue;
    case 256:
      if constexpr (KIND < 2) return launch_gemm<256, KIND>(tmA, tmB, peer, p, grid, stream);
      return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_last_tensor_map_result() { return ds41::last_tensor_map_result(); }

extern "C" int ds41_gemm_tc(const ds41_gemm_args* a, void* stream) {
  if (a == nullptr) return cudaErrorInvalidValue;
  const int M = a->M, N = a->N, K = a->K, batch = a->batch, kind = a->kind, out_mode = a->out_mode;
  const int k_splits = a->k_splits, bn = a->bn;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0 || k_splits <= 0 || kind < 0 || kind > 3 || out_mode < 0 ||
      out_mode > 8)
    return cudaErrorInvalidValue;
  const int elem = kind == 0 ? 2 : 1;
  const int bk = kind == 3 ? 2 * kTileKBytes : kTileKBytes / elem;     // kind 3: two e2m1 values per byte
  const int kb_total = (K + bk - 1) / bk;
  if (1ll * (k_splits - 1) * ((kb_total + k_splits - 1) / k_splits) >= kb_total) return cudaErrorInvalidValue;   // no empty split
  if (kind == 2 && (K % 128 != 0 || a->sfa == nullptr || a->sfb == nullptr)) return cudaErrorInvalidValue;
  if (kind == 3 && (K % 256 != 0 || a->sfa == nullptr || a->sfb == nullptr || a->ag_world > 0 || a->rs_world > 0 ||
                    out_mode == 6 || out_mode == 8 || (bn < 32 && N > bn)))
    return cudaErrorInvalidValue;
  if (kind == 2 && bn < 32 && N > bn) return cudaErrorInvalidValue;      // 16-row scale tiles cannot be lane-shifted
  if (k_splits > 1 && out_mode != 1 && out_mode != 3) return cudaErrorInvalidValue;   // partials are fp32
  if ((out_mode == 4 || out_mode == 5 || out_mode == 8) && a->row_w == nullptr) return cudaErrorInvalidValue;
  if (out_mode == 8 && (bn < 32 || (M & 31) != 0 || k_splits != 1)) return cudaErrorInvalidValue;
  if (out_mode == 7 && (a->scatter_meta == nullptr || a->tile_group == nullptr || (a->ldo & 7) != 0))
    return cudaErrorInvalidValue;
  if (a->tile_group != nullptr && (a->tile_row0 == nullptr || a->tile_end == nullptr || a->n_tiles_dev == nullptr ||
                                   k_splits != 1 || a->max_tiles <= 0))
    return cudaErrorInvalidValue;
  CUtensorMap tmA, tmB;
  const TmaDtype dt = kind == 0 ? TmaDtype::kBF16 : TmaDtype::kU8;
  const bool a_fp4 = a->a_format == 1;
  if (a_fp4 && (kind != 2 || a->ag_world > 0)) return cudaErrorInvalidValue;
  const int a_rows = out_mode == 4 ? a->up_row_offset + M : M;           // dual tiles address gate and up rows
  const int a_batches = a->a_batches > 0 ? a->a_batches : batch;
  const int b_batches = a->b_batch_kind == 1 ? 1 : (a->b_batch_kind == 0 ? a_batches : batch);
  const void* a_base = a->ag_world > 0 ? a->a_peers[a->ag_rank] : a->A;
  // e2m1 operands: strides count elements, two per byte in memory
  cudaError_t e;
  if (kind == 3) {
    // both operands e2m1, packed in memory and in shared memory
    e = make_tensor_map_3d(&tmA, a_base, TmaDtype::kU4x16Align8, K, a_rows, a_batches, a->lda / 2, a->a_batch_stride / 2,
                           bk, kBM, true);
    if (e != cudaSuccess) return e;
    e = make_tensor_map_3d(&tmB, a->B, TmaDtype::kU4x16Align8, K, N, b_batches, a->ldb / 2, a->b_batch_stride / 2, bk, bn,
                           true);
  } else {
    e = a_fp4 ? make_tensor_map_3d(&tmA, a_base, TmaDtype::kU4x16Align16, K, a_rows, a_batches, a->lda / 2,
                                   a->a_batch_stride / 2, bk, kBM, true)
              : make_tensor_map_3d(&tmA, a_base, dt, K, a_rows, a_batches, a->lda * elem, a->a_batch_stride * elem, bk,
                                   kBM, true);
    if (e != cudaSuccess) return e;
    e = make_tensor_map_3d(&tmB, a->B, dt, K, N, b_batches, a->ldb * elem, a->b_batch_stride * elem, bk, bn, true);
  }
  if (e != cudaSuccess) return e;
  StoreMaps peer{};
  int ag_chunks = 1;
  if (a->ag_world > 0) {
    if (a->ag_world > 8 || a->ag_rows <= 0 || a->ag_rows % kBM != 0 || M != a->ag_world * a->ag_rows || batch != 1 ||
        (out_mode > 1 && out_mode != 6) || a->ag_epoch == nullptr || ((1ll * K * elem) & 15) != 0)
      return cudaErrorInvalidValue;
    for (int r = 0; r < a->ag_world; ++r)
      if (a->a_peers[r] == nullptr || a->ag_arrive[r] == nullptr) return cudaErrorInvalidValue;
    // split every 128-row tile into K chunks so that about two rounds of copy units cover the grid
    const int base_units = (a->ag_rows / kBM) * (a->ag_world - 1);
    while (base_units > 0 && base_units * ag_chunks < 2 * sm_count() && ag_chunks < 16 &&
           (1ll * K * elem) % (ag_chunks * 2 * 16) == 0)
      ag_chunks *= 2;
  }
  if (a->rs_world > 0) {
    if (a->rs_world > 8 || a->rs_rows <= 0 || a->rs_rows % kBM != 0 || M != a->rs_world * a->rs_rows || batch != 1 ||
        (out_mode > 1 && out_mode != 6) || k_splits != 1)
      return cudaErrorInvalidValue;
  }
  if (out_mode == 6) {
    if (kind != 0 || bn < 64 || k_splits != 1 || ((a->ldo * 2) & 15) != 0) return cudaErrorInvalidValue;
    if (a->rs_world > 0) {
      // this rank's slot in every destination's buffer: [rs_rows, N] bf16 at slot index rs_rank
      for (int d = 0; d < a->rs_world; ++d) {
        if (a->rs_out[d] == nullptr) return cudaErrorInvalidValue;
        const char* base = static_cast<const char*>(a->rs_out[d]) + 1ll * a->rs_rank * a->rs_rows * a->ldo * 2;
        e = make_tensor_map_3d(&peer.m[d], base, TmaDtype::kBF16, N, a->rs_rows, 1, a->ldo * 2, 0, 64, 32, true);
        if (e != cudaSuccess) return e;
      }
    } else {
      if (a->out == nullptr) return cudaErrorInvalidValue;
      e = make_tensor_map_3d(&peer.m[0], a->out, TmaDtype::kBF16, N, M, batch, a->ldo * 2, a->out_batch_stride * 2, 64,
                             32, true);
      if (e != cudaSuccess) return e;
    }
  }
  GemmParams p{};
  p.ag_world = a->ag_world; p.ag_rank = a->ag_rank; p.ag_rows = a->ag_rows; p.ag_chunks = ag_chunks;
  p.a_row_bytes = a->lda * elem;
  for (int r = 0; r < 8; ++r) {
    p.ag_bufs[r] = r < a->ag_world ? a->a_peers[r] : nullptr;
    p.ag_arrive[r] = r < a->ag_world ? static_cast<uint32_t*>(a->ag_arrive[r]) : nullptr;
  }
  p.ag_epoch = reinterpret_cast<const uint32_t*>(a->ag_epoch);
  p.rs_world = a->rs_world; p.rs_rank = a->rs_rank; p.rs_rows = a->rs_rows;
  for (int r = 0; r < 8; ++r) p.rs_out[r] = r < a->rs_world ? a->rs_out[r] : nullptr;
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.k_splits = k_splits; p.out_mode = out_mode;
  p.ldo = a->ldo; p.out_batch_stride = a->out_batch_stride;
  p.out = k_splits > 1 ? a->split_workspace : a->out;
  if (p.out == nullptr && a->rs_world == 0) return cudaErrorInvalidValue;
  // split planes are laid out [split][batch][rows][ldo]
  const long long plane = (out_mode == 1 ? 1ll * M : 1ll * N) * a->ldo;
  p.out_split_stride = k_splits > 1 ? plane * batch : 0;
  if (k_splits > 1) p.out_batch_stride = plane;
  p.sfa = static_cast<const uint8_t*>(a->sfa);
  p.sfb = static_cast<const uint8_t*>(a->sfb);
  p.sfa_batch_stride = a->sfa_batch_stride;
  p.sfb_batch_stride = a->sfb_batch_stride;
  p.batch_map = a->batch_map;
  p.n_active = a->n_active;
  p.b_batch_kind = a->b_batch_kind;
  p.up_row_offset = a->up_row_offset;
  p.row_w = a->row_w;
  p.row_w_ld = a->row_w_ld;
  p.act_limit = a->act_limit;
  p.tile_group = a->tile_group; p.tile_row0 = a->tile_row0; p.tile_end = a->tile_end; p.n_tiles_dev = a->n_tiles_dev;
  p.wait_flags = reinterpret_cast<const uint32_t* const*>(a->wait_flags);
  p.wait_epoch = reinterpret_cast<const uint32_t*>(a->wait_epoch);
  p.wait_world = a->wait_world;
  p.scatter_meta = reinterpret_cast<const int2*>(a->scatter_meta);
  p.col_limit = a->col_limit;
  for (int r = 0; r < 8; ++r) p.scatter_out[r] = a->scatter_out[r];
  p.static_operand = a->static_operand;
  p.a_fp4 = a_fp4 ? 1 : 0;
  p.alpha = a->alpha != 0.f ? a->alpha : 1.f;
  p.alpha_batch = a->alpha_batch;
  p.sig_counter = a->sig_counter; p.sig_epoch = a->sig_epoch; p.sig_flags = a->sig_flags; p.sig_world = a->sig_world;
  if (p.sig_counter != nullptr && (p.sig_epoch == nullptr || p.sig_flags == nullptr || p.sig_world <= 0 || p.sig_world > 32))
    return cudaErrorInvalidValue;
  p.status = a->status;
  const long long n_t = a->tile_group != nullptr ? a->max_tiles : (N + bn - 1) / bn;
  const long long tiles = 1ll * ((M + kBM - 1) / kBM) * n_t * k_splits * (a->tile_group != nullptr ? 1 : batch);
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (kind) {
    case 0: return dispatch_bn<0>(bn, tmA, tmB, peer, p, grid, s);
    case 1: return dispatch_bn<1>(bn, tmA, tmB, peer, p, grid, s);
    case 2: return dispatch_bn<2>(bn, tmA, tmB, peer, p, grid, s);
    default: return dispatch_bn<3>(bn, tmA, tmB, peer, p, grid, s);
  }
}
