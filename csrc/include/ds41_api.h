// C ABI of libds41_kernels.so.  Every entry point is asynchronous on the given stream, allocates
// nothing, works on caller-owned device buffers and returns a raw cudaError_t value (0 = success).
// Kernels that wait (mbarrier, peer flags) take an `int status[4]` device word: a wait that runs out
// writes {code, where, block, detail} there and the kernel returns instead of hanging.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---------------------------------------------------------------------------------------------------
// Tensor-core GEMM  D[m,n] = sum_k A[m,k] * B[n,k]  (tcgen05 + TMA + TMEM).  Strides in elements.
//   kind      0 bf16, 1 fp8-e4m3 (unscaled), 2 MX fp8 (UE8M0 per 32 elements; scale atoms sfa/sfb)
//   out_mode  0 bf16 [m,n] | 1 f32 [m,n] | 2 bf16 [n,m] | 3 f32 [n,m]
//             4 bf16 [n,m] = silu(min(gate,L)) * clamp(up,-L,L) * row_w[b][n] with gate = A rows [m],
//               up = A rows [up_row_offset + m]   (fused expert FC1)
//             5 f32 [n,m] written only where row_w[b][n] != 0 (expert FC2)
//   k_splits  > 1 writes fp32 planes [split][batch][rows][ldo] into split_workspace (modes 1 and 3)
//   batch_map / n_active: grouped execution - logical batch b uses A batch batch_map[b]; only b < *n_active run
//   b_batch_kind: B batch coordinate 0 = same as A, 1 = always 0 (shared activations), 2 = logical b
typedef struct ds41_gemm_args {
  const void* A;
  const void* B;
  void* out;
  void* split_workspace;
  const void* sfa;
  const void* sfb;
  const int* batch_map;
  const int* n_active;
  const float* row_w;
  int* status;
  long long lda, ldb, ldo;
  long long a_batch_stride, b_batch_stride, out_batch_stride;
  long long sfa_batch_stride, sfb_batch_stride;
  int M, N, K, batch;
  int a_batches;
  int kind, out_mode, k_splits, bn;
  int b_batch_kind;
  int up_row_offset;
  int row_w_ld;
  float act_limit;
  int static_operand;   // 1: A is a weight matrix, 2: B is (prefetched ahead of the stream dependency), 0: neither
  // Fused collectives over NVLink peer memory (out_mode 0/1/6, batch 1):
  //  all-gather -> GEMM (push model): every rank holds a full copy of A (a_peers[r] = rank r's copy, symmetric
  //    memory); rank r wrote its own rows [r*ag_rows, (r+1)*ag_rows) (ag_rows a multiple of 128).  Copier warps of
  //    the kernel push those rows into every peer's copy and bump the peer's arrival counters
  //    ag_arrive[d][src * ag_rows/128 + tile]; the TMA producer loads a remote tile from LOCAL memory once its counter
  //    has reached *ag_epoch * chunks (bounded wait).  Counters only grow; *ag_epoch is the call count.
  //  GEMM -> reduce-scatter: the output rows owned by rank d (rs_rows each) are stored into rs_out[d] at row
  //    rs_rank * rs_rows + local_row, i.e. every destination receives one slot per source rank to sum in fixed order.
  //    With out_mode 6 the slots are bf16 and written by TMA stores from shared memory.
  //  out_mode 6 without rs_world: bf16 [m,n] output through the same TMA-store epilogue (bn >= 64, bf16 kind).
  int ag_world, ag_rank, ag_rows;
  int rs_world, rs_rank, rs_rows;
  void* a_peers[8];
  void* ag_arrive[8];
  const void* ag_epoch;      // device word
  void* rs_out[8];
  // Grouped tokens (expert-parallel prefill; swap-AB, B = flat rows sorted by expert, B batch kind 1):
  //   device tile table: tile j = rows [tile_row0[j], tile_end[j]) of expert tile_group[j]; *n_tiles_dev live tiles,
  //   at most max_tiles.  row_w is then indexed by flat row.  out_mode 7 scatters result rows (bf16) to
  //   scatter_out[meta.x] + meta.y * ldo, meta = scatter_meta[row] (P2P stores: the combine half of the all-to-all).
  //   wait_flags / wait_epoch / wait_world: peers whose stores this GEMM consumes (bounded wait before the first load).
  const int* tile_group;
  const int* tile_row0;
  const int* tile_end;
  const int* n_tiles_dev;
  const void* scatter_meta;
  const void* wait_flags;
  const void* wait_epoch;
  void* scatter_out[8];
  int max_tiles;
  int wait_world;
  // kind 2 only: 1 = A holds e2m1 (FP4) values, two per byte in memory (even element in the low nibble), with UE8M0
  // scales per 32 elements; lda / a_batch_stride then count elements.  B stays e4m3.
  int a_format;
  // out_mode 8 (indexer scores): M rows are (query, head) pairs with 32 heads per query; out is fp32 [M/32, ldo];
  // row_w[query * row_w_ld + head] weights relu(acc); columns >= col_limit[query] (if given) are written as -inf.
  const int* col_limit;
  // kind 3 (NVFP4 x NVFP4): A and B hold e2m1 values two per byte, sfa / sfb hold E4M3 scales per 16 elements in
  // 512-byte atoms of (128 rows, 64 K elements): byte = (row%32)*16 + ((row/32)%4)*4 + (k/16)%4, atoms [row/128][K/64].
  // K must be a multiple of 256; lda / ldb / batch strides count elements; alpha (the product of the two global
  // scales, 0 = 1) multiplies the accumulators.
  float alpha;
  const float* alpha_batch;   // optional: one more factor per A batch (a global scale per expert)
  // Completion signal folded into the kernel (multi-rank decode): the CTA that finishes last bumps *sig_epoch and
  // stores the new value to sig_flags[0 .. sig_world) (device array of flag addresses, one slot in every rank's
  // memory), with release semantics at system scope.  sig_counter is a zeroed device word, left at zero again.
  unsigned int* sig_counter;
  unsigned int* sig_epoch;
  unsigned int* const* sig_flags;
  int sig_world;
} ds41_gemm_args;

int ds41_gemm_tc(const ds41_gemm_args* args, void* stream);

// ---------------------------------------------------------------------------------------------------
// Hyper-connections and embedding (hc.cu)
int ds41_embed_streams(const int* tokens, const void* embed, void* streams, float* pre, int rows, int H, int mult,
                       int vocab, void* stream);
// part_bases: HOST array of n_ranks device pointers (fp32 planes [n_splits][rows][H], local or peer memory);
// wait_flags: DEVICE array of n_ranks flag pointers, wait_epoch: device word holding the value to wait for.
int ds41_hc_post_mix(const void* streams_in, void* streams_out, const float* const* part_bases, int n_ranks,
                     int n_splits, long long split_stride, const float* post, const float* comb, const float* fn,
                     float* partial, int rows, int H, const uint32_t* const* wait_flags, const uint32_t* wait_epoch,
                     int* status, const float* pre_in, const float* norm_w, void* xn, float* tap_mean, float norm_eps,
                     void* stream);
int ds41_hc_finish(const float* partial, int n_slices, const float* scale, const float* base, const float* pre_in,
                   const void* streams, const float* norm_w, float* next_pre, float* post, float* comb, void* xn,
                   float* tap_mean, void* xq, void* xq_sf, int rows, int H, int iters, float hc_eps, float norm_eps,
                   const float* mix_planes, int mix_splits, long long mix_split_stride, int mix_ld, void* stream);
// hc_post_mix with fn == NULL only expands, stores and leaves row r's sum of squares in partial[r * 25 + 24] (a
// single slice: hc_finish is then called with n_slices = 1); the 24 mixes
// projections then come from a GEMM of the stored streams [rows, 4H] with the matrix as bf16 high and low parts
// (columns j and 24 + j of fp32 split-K planes [mix_splits][rows][mix_ld]), which hc_finish reads as `mix_planes`
// (NULL: the projections are in `partial`).  In that form hc_post_mix can also collapse and normalise the row it holds
// (xn != NULL with pre_in, optional norm_w / tap_mean): hc_finish is then called with xn == NULL and only turns the
// projections into next_pre / post / comb.

// Fused small-batch step (hc_step.cu): expand with the sublayer's partial planes, next mixes, collapse with the
// known `pre_in`, RMSNorm (+ optional E4M3/scale-atom output) in one launch.  part_bases: HOST array of device
// pointers; wait_flags: DEVICE array of peer flag pointers.  `tickets` [rows] must be zero before the first call.
typedef struct ds41_hc_step_args {
  const void* streams_in;
  void* streams_out;
  const float* const* part_bases;
  const float* post;
  const float* comb;
  const float* pre_in;
  const float* fn;
  const float* scale;
  const float* base;
  const float* norm_w;
  float* partial;        // [H/128][rows][26]
  float* xc;             // [rows][H]
  float* next_pre;
  float* post_out;
  float* comb_out;
  void* xn;
  float* tap_mean;
  void* xq;
  void* xq_sf;
  unsigned int* tickets;
  const uint32_t* const* wait_flags;
  const uint32_t* wait_epoch;
  int* status;
  long long split_stride;
  int n_ranks, n_splits;
  int rows, H, iters;
  float hc_eps, norm_eps;
} ds41_hc_step_args;
int ds41_hc_step(const ds41_hc_step_args* args, void* stream);

// ---------------------------------------------------------------------------------------------------
// Attention-side projections' epilogues and cache writes (attn_ops.cu)
// kv_row_bytes (qkv_post, compress, attend): 0 = latent rows are bf16 [D]; otherwise FP8 rows of that many bytes:
// D e4m3 values, then D/32 UE8M0 scales (ceil_pow2(amax/448) per 32 elements), padded to a multiple of 16 bytes.
int ds41_qkv_post(const float* planes, int splits, int rows, int ntot, int Q, int D, int rope_dim, int extra_f32,
                  int index_heads, float index_scale, const float* q_norm_w, const float* kv_norm_w,
                  const float* inv_freq, const int* row_pos, const int* row_slot, void* q_lat, void* win, int ring,
                  float* extras, float eps, int kv_row_bytes, void* stream);
int ds41_compress(const float* extras, int extra_stride, int rows, int D, int ID, int rope_dim, int ratio,
                  const int* row_pos, const int* row_slot, float* pending, const float* comp_norm_w, const void* wk,
                  const float* k_norm_w, const float* inv_freq, const float* inv_freq_idx, const int* page_table,
                  int max_pages, int page_rows, void* comp_pool, void* idx_pool, float eps, int kv_row_bytes,
                  int idx_row_bytes, void* stream);

// ---------------------------------------------------------------------------------------------------
// Indexer, top-k and sparse attention (sparse_attn.cu)
// idx_row_bytes (ds41_compress, ds41_index_score_cand, ds41_index_prepare): 0 = index keys are bf16 rows of ID values;
// > 0 = FP4 rows that many bytes apart: ID/2 bytes of E2M1 pairs (even value in the low nibble), then ID/32 UE8M0
// scales (68 bytes for ID = 128).  With FP4 keys the queries are quantised to the same format before the dot.
int ds41_index_score(const void* q, long long ldq, int q_off, const float* w, int w_stride, int w_off,
                     const void* idx_pool, const int* page_table, int max_pages, int page_rows, const int* row_pos,
                     const int* row_slot, const float* inv_freq_idx, int rows, int IH, int ID, int ratio,
                     float* scores, int max_keys, void* stream);
// Operands of the tensor-core indexer (one request per pass): RoPE'd queries [rows*IH, ID], the request's keys gathered
// into [n_keys, ID], visible keys per row.  The scores then come from ds41_gemm_tc with out_mode 8.
int ds41_index_prepare(const void* q, long long ldq, int q_off, const void* idx_pool, const int* page_table,
                       int max_pages, int page_rows, const int* row_pos, const int* row_slot,
                       const float* inv_freq_idx, int rows, int IH, int ID, int ratio, int n_keys, int max_keys,
                       void* qr, void* kc, int* n_vis, int idx_row_bytes, void* stream);
int ds41_topk_select(const float* scores, int max_keys, const int* row_pos, const int* row_slot, int ratio, int k,
                     int* sel, int* n_sel, int rows, void* stream);
// Candidate blocks of the long-context indexer: ds41_candidate_select reduces one layer's scores to block maxima (blocks
// of `block` keys, the newest visible block pinned), keeps the best `k_blocks` blocks per row and publishes them as a list
// [rows, k_blocks] and a bit mask [rows, words] (32 * words * block >= max_keys).  The *_cand variants of the score and
// top-k kernels skip / exclude keys whose block bit is 0 (cand_mask null = unrestricted).
int ds41_candidate_select(const float* scores, int max_keys, const int* row_pos, const int* row_slot, int ratio,
                          int block, int k_blocks, int* blocks, int* n_blocks, void* mask, int words, int rows,
                          void* stream);
int ds41_index_score_cand(const void* q, long long ldq, int q_off, const float* w, int w_stride, int w_off,
                          const void* idx_pool, const int* page_table, int max_pages, int page_rows,
                          const int* row_pos, const int* row_slot, const float* inv_freq_idx, int rows, int IH, int ID,
                          int ratio, float* scores, int max_keys, const void* cand_mask, int cand_words,
                          int cand_block, int idx_row_bytes, void* stream);
int ds41_topk_select_cand(const float* scores, int max_keys, const int* row_pos, const int* row_slot, int ratio, int k,
                          int* sel, int* n_sel, int rows, const void* cand_mask, int cand_words, int cand_block,
                          void* stream);
int ds41_attend(const void* q, long long ldq, int q_off, int rows, int heads, int D, int window, int ring,
                const int* row_pos, const int* row_slot, const void* win, const void* comp_pool, const int* sel,
                const int* n_sel, int k, const int* page_table, int max_pages, int page_rows, const float* inv_freq,
                int rope_dim, float scale, int n_splits, const int* row_hi, float* part_o, float* part_ml,
                const float* sink, void* out, long long ldo, int kv_row_bytes, void* stream);

// ---------------------------------------------------------------------------------------------------
// Router / experts (moe.cu)
int ds41_router_select(const float* planes, int splits, int rows, int ntot, int E, int I_sh, int topk,
                       const float* bias, float route_scale, float limit, int* ids, float* weights, void* shared_act,
                       void* stream);
int ds41_moe_plan(const int* ids, const float* weights, const int* row_slot, int rows, int topk, int e0, int e1,
                  int max_active, int row_w_ld, int* active, int* n_active, float* row_w, int* slot_of,
                  void* stream);
int ds41_moe_combine(const float* fc2, const int* slot_of, const float* shared, int shared_splits, int rows,
                     int topk, int H, float* out, void* stream);
int ds41_signal(uint32_t* epoch, uint32_t* flag, void* stream);
// bump *epoch and store it to flags[0 .. n) (a device array of flag addresses in this and the peers' memory): every
// rank then polls flags in its own memory
int ds41_signal_all(uint32_t* epoch, uint32_t* const* flags, int n, void* stream);
// ds41_moe_combine with the completion signal of ds41_signal_all folded in (done by the block that finishes last;
// `counter` is a zeroed device word, left at zero again)
int ds41_moe_combine_signal(const float* fc2, const int* slot_of, const float* shared, int shared_splits, int rows,
                            int topk, int H, float* out, unsigned int* counter, uint32_t* epoch,
                            uint32_t* const* flags, int n_flags, void* stream);
int ds41_reduce_planes(const float* planes, int splits, long long plane, void* out, int as_bf16, long long n,
                       void* stream);
// planes [split][group][rows][width] fp32 (split-K partials of a grouped projection) -> bf16 out [rows][ld_out],
// group g in columns [g * width, (g + 1) * width)
int ds41_reduce_groups(const float* planes, int splits, int groups, int rows, int width, void* out, long long ld_out,
                       void* stream);

// ---------------------------------------------------------------------------------------------------
// Head epilogues (sampler.cu)
int ds41_argmax_rows(const float* logits, long long ld, int rows, int vocab_local, int vocab_offset,
                     const uint32_t* mask, int mask_words, float* best_val, int* best_idx, int* row_status,
                     void* stream);
int ds41_argmax_merge(const float* const* vals, const int* const* idxs, int n_ranks, int rows, int* out,
                      const uint32_t* const* wait_flags, const uint32_t* wait_epoch, int* status, void* stream);
int ds41_decode_feedback(const int* chosen, int* tokens, int* pos, int rows, void* stream);
int ds41_spec_accept(const int* inputs, const int* chosen, const int* first, const int* count, int reqs,
                     int max_emit, int eos, int* accepted, int* emit, int* n_emit, void* stream);

// ---------------------------------------------------------------------------------------------------
// Collective epilogues (comm.cu).  slots: fp32 [world][n] (one slot per source rank), summed in rank order.
int ds41_rs_reduce(const float* slots, int world, long long slot_stride, void* out, int as_bf16, long long n,
                   const void* wait_flags, const void* wait_epoch, int* status, void* stream);

// ---------------------------------------------------------------------------------------------------
// dSpark drafter support (dspark.cu)
int ds41_taps_pack(const float* taps, void* out, int n_taps, int rows, int H, long long tap_stride, void* stream);
int ds41_norm_rows(const float* planes, int splits, long long plane, const float* w, void* out, int rows, int N,
                   float eps, void* stream);
// Draft sampling parameters of ds41_markov_step (null = greedy): Gumbel-max over x / temperature with Philox uniforms
// addressed by (seed, subsequence, offset + token / 4, token % 4).
typedef struct {
  float temperature;
  unsigned long long seed, subsequence, offset;
} ds41_draft_rng;
int ds41_markov_step(const float* logits, const void* head, const void* embed, const int* prev_token, int v_local,
                     int v_offset, int rank, int vocab, float* block_val, int* block_idx, int n_blocks,
                     unsigned int* ticket, float* best_val, int* best_idx, const ds41_draft_rng* rng, void* stream);
// Confidence head of the drafter: out[j] = weight . [hidden[j] (fp32, H) | embed[prev_j] (bf16, rank)], raw (no sigmoid);
// prev_0 = anchor[0], prev_j = drafts[j - 1].
int ds41_dspark_confidence(const float* hidden, long long ld_hidden, const void* embed, int rank, const int* anchor,
                           const int* drafts, const void* weight, float* out, int rows, int H, int vocab, void* stream);
int ds41_spec_feedback(const int* inputs, const int* chosen, int width, int forced_accept, int eos, int* accepted,
                       int* emitted, int* n_emitted, int* next_anchor, int* target_pos, int* draft_pos,
                       int* draft_hi, int* target_tokens, int* draft_tokens, long long* total_emitted, void* stream);
int ds41_copy_ints(const int* src, int* dst, int n, void* stream);

// ---------------------------------------------------------------------------------------------------
// Quantisation (quant.cu).  sf: scale atoms [batch][ceil(rows/128)][K/128][512]; group 32 or 128.
int ds41_act_quant_mx(const void* x, long long ldx, long long x_batch_stride, void* q, long long ldq,
                      long long q_batch_stride, void* sf, long long sf_batch_stride, int rows, int K, int batch,
                      int group, const int* n_active, void* stream);

// ---------------------------------------------------------------------------------------------------
// Expert-parallel token exchange over peer memory (ep.cu).  Pointer tables hold one pointer per rank (symmetric memory).
typedef struct {
  int world, rank, e_local, topk, tokens, H, cap, bn, bn2, max_tiles;   // bn2 > 0: second tile table of bn2-row tiles
  const void* x;            // [tokens, H] bf16 rows of this rank
  const int* ids;           // [tokens, topk] global expert ids (out of range = no route)
  const float* weights;     // [tokens, topk]
  uint32_t* epoch;          // rank-local step counter (bumped by ds41_ep_count)
  int* cursor;              // [world * e_local] scratch
  int* ticket;              // [1] scratch
  void* counts[8];          // int [world(src)][e_local] at each rank
  void* send_base[8];       // int [world(dst)][e_local] at each rank
  void* recv_x[8];          // bf16 [cap, H] at each rank
  void* recv_meta[8];       // int2 [cap] {source rank, token*topk+k}
  void* recv_w[8];          // float [cap]
  void* flags[8];           // uint32 [4] phase flags at each rank
  int* tile_group;          // [2 * max_tiles] tile tables of the grouped GEMMs (local): bn tiles, then bn2 tiles
  int* tile_row0;
  int* tile_end;
  int* n_tiles;             // [2]
  int* total_rows;
  int* status;
  // FP8 rows on the wire (optional, all three set or none): ds41_ep_dispatch quantises every row it sends (E4M3 values,
  // one UE8M0 scale per 128 values) and stores values and scales straight into the destination's operand buffers of
  // the block-scaled FC1 - 5280 bytes per row of 5120 values instead of 10240 - and recv_x is not written.
  void* recv_q[8];          // uint8 [cap, H] at each rank
  void* recv_sf[8];         // scale atoms [cap/128][H/128][512] at each rank
  int wire_fp8;
} ds41_ep_args;
int ds41_ep_count(const ds41_ep_args* a, void* stream);
int ds41_ep_plan(const ds41_ep_args* a, void* stream);
int ds41_ep_dispatch(const ds41_ep_args* a, int blocks, void* stream);
int ds41_ep_mark(const ds41_ep_args* a, int phase, void* stream);
int ds41_ep_wait(const ds41_ep_args* a, int phase, void* stream);
int ds41_ep_combine(const ds41_ep_args* a, const void* comb, const float* extra, long long extra_ld, void* out,
                    int as_bf16, void* stream);

// ---------------------------------------------------------------------------------------------------
// Token sampler (sampler_rows.cu): one 64-byte parameter block per row.  Status per row: 0 ok, 1 no candidate,
// 2 non-finite logit, 3 bad temperature, 5 internal, 6 bad parameter (same codes as ds41_sample_token on the host).
typedef struct {
  float temperature;
  int top_k;                    // <= 0: off
  float top_p;                  // >= 1: off
  float min_p;                  // <= 0: off
  unsigned long long seed;
  unsigned long long position;  // absolute index of the emitted token
  int mask_row;                 // row of the packed allow-mask arena, < 0: no mask
  int reserved[7];
} ds41_sample_row;
int ds41_sample_rows(const float* logits, long long ld, int rows, int vocab, const uint32_t* masks, int mask_words,
                     const ds41_sample_row* params, int* tokens, int* status, void* stream);

// ds41_attend with a per-row floor on the window: positions below row_lo[r] are not attended (a window that was
// rebuilt from that position on, e.g. the decoder layers after a prompt's tail replay); row_lo null = no floor.
int ds41_attend_floor(const void* q, long long ldq, int q_off, int rows, int heads, int D, int window, int ring,
                      const int* row_pos, const int* row_slot, const void* win, const void* comp_pool, const int* sel,
                      const int* n_sel, int k, const int* page_table, int max_pages, int page_rows,
                      const float* inv_freq, int rope_dim, float scale, int n_splits, const int* row_hi, float* part_o,
                      float* part_ml, const float* sink, void* out, long long ldo, int kv_row_bytes, const int* row_lo,
                      void* stream);

// ds41_attend_floor with FP4 compressed rows: comp_row_bytes > 0 says that comp_pool holds FP4 rows (D/2 e2m1 bytes, then
// D/16 E4M3 scales, padded to comp_row_bytes) while the window rows are FP8 rows of kv_row_bytes; 0 = one format.
int ds41_attend_kv(const void* q, long long ldq, int q_off, int rows, int heads, int D, int window, int ring,
                   const int* row_pos, const int* row_slot, const void* win, const void* comp_pool, const int* sel,
                   const int* n_sel, int k, const int* page_table, int max_pages, int page_rows, const float* inv_freq,
                   int rope_dim, float scale, int n_splits, const int* row_hi, float* part_o, float* part_ml,
                   const float* sink, void* out, long long ldo, int kv_row_bytes, int comp_row_bytes, const int* row_lo,
                   void* stream);

// Sparse attention on the tcgen05 tensor cores (attend_tc.cu): same semantics as ds41_attend_kv for D = 512 or 128 and at
// most 64 heads.  A persistent grid walks the (row, key split) items; each item multiplies every head against each
// gathered 64-key tile.  With n_splits == 1 the kernel writes the final bf16 rows itself (sink, normalisation, inverse
// RoPE), otherwise partials go to part_o / part_ml and ds41_attend_merge finishes them.  Waits are bounded; `status`
// receives {code, site, row, detail}.
typedef struct {
  const void* q;
  long long ldq;
  int q_off;
  int rows, heads, D, window, ring;
  const int* row_pos;
  const int* row_slot;
  const int* row_hi;
  const int* row_lo;
  const void* win;
  const void* comp_pool;
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
  void* out;
  long long ldo;
  int kv_row_bytes, comp_row_bytes;
  int* status;
} ds41_attend_args;
int ds41_attend_tc(const ds41_attend_args* args, void* stream);
// Merge of split-key partials: part_o [rows][n_splits][heads][D] fp32, part_ml [rows][n_splits][heads][2] = (max, sum).
int ds41_attend_merge(const float* part_o, const float* part_ml, const float* sink, const int* row_pos,
                      const int* row_slot, const float* inv_freq, int rope_dim, int heads, int D, int n_splits, int rows,
                      void* out, long long ldo, void* stream);

// ---------------------------------------------------------------------------------------------------
// Pipeline-stage handoff over peer memory (pp.cu).  Counters are 32-bit words in symmetric memory; every wait is bounded
// and reports {flag timeout, site} in the status word.
int ds41_pp_signal(void* flag, unsigned value, void* stream);
int ds41_pp_wait(const void* flag, unsigned value, int* status, int site, void* stream);
int ds41_pp_pull(const void* src, void* dst, long long nbytes, const void* flag, unsigned value, int* status, int site,
                 void* stream);

// ---------------------------------------------------------------------------------------------------
// Engram memory (engram.cu): table rows (dim e4m3 values + dim/32 UE8M0 scales, row_bytes apart) -> bf16 [n_rows, dim];
// gated residual update of the 4 streams from kv = [rows][4 keys + 1 value][H] (bf16); text_mask 0 = pass through.
int ds41_engram_dequant(const void* rows_q, int row_bytes, int dim, void* out, int n_rows, void* stream);
int ds41_engram_gate(const void* x, const void* kv, const void* q_w, const void* k_w, const uint8_t* text_mask,
                     void* out, int rows, int H, float eps, void* stream);
// Rows of a table converted to NVFP4 (dim/2 bytes of E2M1 pairs + dim/16 E4M3 scales per record, one fp32 scale per
// table) -> bf16((code * scale) * table_scale).
int ds41_engram_dequant_nvfp4(const void* rows_q, int row_bytes, int dim, float table_scale, void* out, int n_rows,
                              void* stream);

// ---------------------------------------------------------------------------------------------------
// Hidden-state rows as wire records (wire.cu): H E4M3 values + H/32 UE8M0 scales per row, `row_bytes` apart
// (multiple of 8, >= H + H/32); bf16 side with leading dimension ld (multiple of 8).  Both pointers 16-byte aligned.
int ds41_wire_encode(const void* x, long long ldx, void* out, long long row_bytes, int rows, int H, void* stream);
int ds41_wire_decode(const void* in, long long row_bytes, void* y, long long ldy, int rows, int H, void* stream);

// ---------------------------------------------------------------------------------------------------
// Vision tower elementwise kernels (vision.cu); all tensors bf16 unless noted.
int ds41_vis_rmsnorm(const void* x, const void* w, void* out, int rows, int W, float eps, void* stream);
int ds41_vis_bias_act(const void* x, const void* bias, const void* residual, void* out, long long rows, int cols,
                      int act, void* stream);
int ds41_vis_silu_mul(const void* gu, void* out, int rows, int I, void* stream);
int ds41_vis_rope2d(void* qkv, const int* pos_hw, int rows, int W, int heads, float theta, void* stream);
int ds41_vis_softmax(const float* s, long long ld, long long rows, int n_valid, float scale, void* p, long long ldp,
                     int n_pad, void* stream);
int ds41_vis_merge(const void* x, void* out, int gh, int gw, int m, int W, void* stream);
int ds41_vis_scatter(const void* src, const int* rows, void* dst, int n, int H, int copies, void* stream);

// Prefill-sized activation quantiser (1x128 scales, one warp per row); rows >= *rows_dev (if given) are skipped.
int ds41_act_quant_mx_rows(const void* x, long long ldx, void* q, long long ldq, void* sf, int rows, int K,
                           const int* rows_dev, void* stream);

// NVFP4 activation rows (e2m1 two per byte + E4M3 scale atoms per 16 elements, relative to global_scale); ldq counts
// elements; rows >= *rows_dev (if given) are skipped; `batch` row blocks of `rows` rows each (strides in elements of x / q
// and bytes of sf), of which only the first *n_active (if given) are processed.
int ds41_act_quant_nvfp4_rows(const void* x, long long ldx, void* q, long long ldq, void* sf, int rows, int K,
                              float global_scale, const int* rows_dev, int batch, long long x_batch_stride,
                              long long q_batch_stride, long long sf_batch_stride, const int* n_active, void* stream);

#ifdef __cplusplus
}
#endif
