// Vocabulary-head epilogues: masked greedy argmax, cross-shard merge, speculative accept.
//
//  argmax_rows   : per row, (max logit, lowest token id) over this rank's vocabulary shard under an optional
//                  packed allow-mask (bit set = allowed), non-finite logits reported through a status word
//                  (greedy contract of native/cuda/kernels/v41_sampling_gpu.cu:303-323)
//  argmax_merge  : deterministic merge of the per-shard candidates (highest value, lowest id)
//                  (native/include/ds41rt_v41_dspark.h:21-34)
//  spec_accept   : accept-prefix rule of speculative verification: draft j is accepted while it equals the
//                  target's choice after draft j-1; emits accepted count and the tokens to emit
//                  (rust/crates/ds41rt-core/src/dspark_verify.rs:18-52)
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

struct ArgmaxParams {
  const float* logits;    // [rows][ld]
  long long ld;
  int vocab_local, vocab_offset;
  const uint32_t* mask;   // optional [rows][mask_words] over the GLOBAL vocabulary
  int mask_words;
  float* best_val;        // [rows]
  int* best_idx;          // [rows] global token id
  int* row_status;        // optional [rows]: 1 = non-finite logit seen, 2 = no allowed candidate
};

__global__ void __launch_bounds__(1024) argmax_rows_kernel(ArgmaxParams p) {
  __shared__ float wv[32];
  __shared__ int wi[32];
  __shared__ int bad;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();
  if (tid == 0) bad = 0;
  __syncthreads();
  float v = -INFINITY;
  int idx = 0x7fffffff;
  int nonfinite = 0;
  const float* row = p.logits + 1ll * r * p.ld;
  const uint32_t* mrow = p.mask != nullptr ? p.mask + 1ll * r * p.mask_words : nullptr;
  auto take = [&](int i, float x) {
    const int tok = p.vocab_offset + i;
    if (!isfinite(x)) nonfinite = 1;
    bool ok = true;
    if (mrow != nullptr) ok = (mrow[tok >> 5] >> (tok & 31)) & 1u;
    if (ok && (x > v || (x == v && tok < idx))) { v = x; idx = tok; }
  };
  if ((p.ld & 3) == 0 && (reinterpret_cast<uintptr_t>(p.logits) & 15) == 0) {
    // 16-byte loads, two of them in flight per thread: a row is half a megabyte read by one block
    const int n4 = p.vocab_local >> 2;
    for (int g = tid; g < n4; g += 2048) {
      const float4 a = *reinterpret_cast<const float4*>(row + 4 * g);
      const bool second = g + 1024 < n4;
      const float4 b = second ? *reinterpret_cast<const float4*>(row + 4 * (g + 1024)) : make_float4(0.f, 0.f, 0.f, 0.f);
      take(4 * g, a.x); take(4 * g + 1, a.y); take(4 * g + 2, a.z); take(4 * g + 3, a.w);
      if (second) {
        const int h = 4 * (g + 1024);
        take(h, b.x); take(h + 1, b.y); take(h + 2, b.z); take(h + 3, b.w);
      }
    }
    for (int i = 4 * n4 + tid; i < p.vocab_local; i += 1024) take(i, row[i]);
  } else {
    for (int i = tid; i < p.vocab_local; i += 1024) take(i, row[i]);
  }
  if (nonfinite) bad = 1;
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  if (lane == 0) { wv[warp] = v; wi[warp] = idx; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 32; ++w)
      if (wv[w] > v || (wv[w] == v && wi[w] < idx)) { v = wv[w]; idx = wi[w]; }
    p.best_val[r] = v;
    p.best_idx[r] = idx == 0x7fffffff ? -1 : idx;
    if (p.row_status != nullptr) p.row_status[r] = bad ? 1 : (idx == 0x7fffffff ? 2 : 0);
  }
}

// candidates from `n_ranks` shards: vals[k][rows], idxs[k][rows] (pointer tables, possibly peer memory)
struct MergeArgs {
  const float* vals[8];
  const int* idxs[8];
  int n_ranks, rows;
  int* out;     // [rows]
  const uint32_t* const* wait_flags;   // optional device array of n_ranks flag pointers
  const uint32_t* wait_epoch;
  int* status;
};
__global__ void argmax_merge_kernel(MergeArgs p) {
  pdl_launch_dependents();
  pdl_wait();
  if (p.wait_flags != nullptr && p.n_ranks > 1) {
    if (threadIdx.x < p.n_ranks) flag_wait_ge(p.wait_flags[threadIdx.x], *p.wait_epoch, p.status, 500 + threadIdx.x);
    __syncthreads();
  }
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= p.rows) return;
  float v = -INFINITY;
  int idx = -1;
  // every rank's candidate is requested before the first comparison: a peer load takes a few microseconds
  for (int k0 = 0; k0 < p.n_ranks; k0 += 8) {
    float ovs[8];
    int ois[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      ovs[u] = -INFINITY;
      ois[u] = -1;
      if (k0 + u < p.n_ranks) { ovs[u] = p.vals[k0 + u][r]; ois[u] = p.idxs[k0 + u][r]; }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float ov = ovs[u];
      const int oi = ois[u];
      if (oi >= 0 && (idx < 0 || ov > v || (ov == v && oi < idx))) { v = ov; idx = oi; }
    }
  }
  p.out[r] = idx;
}

// Verification chunk of request q occupies rows [first[q], first[q] + n[q]): row 0 carries the anchor token,
// row j the j-th draft.  chosen[row] is the target's token AFTER consuming that row's input.
// accepted[q] = number of drafts accepted; emit[q][0..accepted] = chosen tokens of rows 0..accepted.
struct AcceptParams {
  const int* inputs;    // [rows] token fed at each row
  const int* chosen;    // [rows]
  const int* first;     // [reqs]
  const int* count;     // [reqs]
  int reqs, max_emit, eos;
  int* accepted;        // [reqs]
  int* emit;            // [reqs][max_emit]
  int* n_emit;          // [reqs]
};
__global__ void spec_accept_kernel(AcceptParams p) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (q >= p.reqs) return;
  const int f = p.first[q], n = p.count[q];
  int acc = 0;
  int emitted = 0;
  for (int j = 0; j < n; ++j) {
    const int tok = p.chosen[f + j];
    if (emitted < p.max_emit) p.emit[q * p.max_emit + emitted] = tok;
    ++emitted;
    if (tok == p.eos) break;                                  // stop token ends the chunk
    if (j + 1 < n && p.inputs[f + j + 1] == tok) ++acc;       // next draft matches -> keep going
    else break;
  }
  p.accepted[q] = acc;
  p.n_emit[q] = min(emitted, p.max_emit);
}

// Device-side feedback for back-to-back decode steps: next input token = chosen token, position + 1.
__global__ void decode_feedback_kernel(const int* chosen, int* tokens, int* pos, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (r < rows) {
    tokens[r] = chosen[r];
    pos[r] += 1;
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_decode_feedback(const int* chosen, int* tokens, int* pos, int rows, void* stream) {
  if (rows <= 0) return cudaErrorInvalidValue;
  return launch_pdl(decode_feedback_kernel, dim3((rows + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream),
                    chosen, tokens, pos, rows);
}

extern "C" int ds41_argmax_rows(const float* logits, long long ld, int rows, int vocab_local, int vocab_offset,
                                const uint32_t* mask, int mask_words, float* best_val, int* best_idx,
                                int* row_status, void* stream) {
  if (rows <= 0 || vocab_local <= 0) return cudaErrorInvalidValue;
  ArgmaxParams p{logits, ld, vocab_local, vocab_offset, mask, mask_words, best_val, best_idx, row_status};
  return launch_pdl(argmax_rows_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_argmax_merge(const float* const* vals, const int* const* idxs, int n_ranks, int rows, int* out,
                                 const uint32_t* const* wait_flags, const uint32_t* wait_epoch, int* status,
                                 void* stream) {
  if (n_ranks <= 0 || n_ranks > 8 || rows <= 0) return cudaErrorInvalidValue;
  MergeArgs p{};
  for (int k = 0; k < n_ranks; ++k) { p.vals[k] = vals[k]; p.idxs[k] = idxs[k]; }
  p.n_ranks = n_ranks; p.rows = rows; p.out = out;
  p.wait_flags = wait_flags; p.wait_epoch = wait_epoch; p.status = status;
  return launch_pdl(argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int ds41_spec_accept(const int* inputs, const int* chosen, const int* first, const int* count, int reqs,
                                int max_emit, int eos, int* accepted, int* emit, int* n_emit, void* stream) {
  if (reqs <= 0 || max_emit <= 0) return cudaErrorInvalidValue;
  AcceptParams p{inputs, chosen, first, count, reqs, max_emit, eos, accepted, emit, n_emit};
  return launch_pdl(spec_accept_kernel, dim3((reqs + 63) / 64), dim3(64), 0, static_cast<cudaStream_t>(stream), p);
}
