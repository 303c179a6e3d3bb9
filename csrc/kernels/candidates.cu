// Candidate-block plumbing of the long-context indexer.
//
// At the candidate layer the lightning-indexer scores of all compressed positions are reduced to one score per block
// of `block` consecutive positions (block_max); the top blocks are selected with the ordinary top-k kernel; the later
// index layers then score only the positions of those blocks (expand_blocks turns block ids into position lists,
// clipped to the causal limit of the row).
//   block_max     : scores [rows, ld] (fp32, -inf = not visible) -> out [rows, ceil(n_keys / block)]
//   expand_blocks : blocks [rows, k] (block ids, -1 = empty) -> pos [rows, k * block] (position or -1), count per row
// Reference: native/cuda/kernels/v41_candidate_blocks.cu:13,18,39 (block-max, expand, tile positions).
#include "ds41_api.h"
#include "ds41_launch.cuh"

namespace ds41 {

__global__ void __launch_bounds__(256)
block_max_kernel(const float* __restrict__ scores, long long ld, int n_keys, int block, float* __restrict__ out,
                 int n_blocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  const float* s = scores + 1ll * r * ld + 1ll * b * block;
  float m = -INFINITY;
  for (int j = 0; j < block && b * block + j < n_keys; ++j) m = fmaxf(m, s[j]);
  out[1ll * r * n_blocks + b] = m;
}

__global__ void __launch_bounds__(256)
expand_blocks_kernel(const int* __restrict__ blocks, int k, int block, const int* __restrict__ limit,
                     int* __restrict__ pos, int* __restrict__ count) {
  __shared__ int s_count;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  const int lim = limit != nullptr ? limit[r] : 0x7fffffff;      // positions >= lim are not visible to this row
  int mine = 0;
  for (int i = threadIdx.x; i < k * block; i += blockDim.x) {
    const int b = blocks[1ll * r * k + i / block];
    int p = b < 0 ? -1 : b * block + i % block;
    if (p >= lim) p = -1;
    pos[1ll * r * k * block + i] = p;
    mine += p >= 0;
  }
  atomicAdd(&s_count, mine);
  __syncthreads();
  if (threadIdx.x == 0 && count != nullptr) count[r] = s_count;
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_block_max(const float* scores, long long ld, int rows, int n_keys, int block, float* out,
                              void* stream) {
  if (scores == nullptr || out == nullptr || rows <= 0 || n_keys <= 0 || block <= 0) return cudaErrorInvalidValue;
  const int n_blocks = (n_keys + block - 1) / block;
  return launch_pdl(block_max_kernel, dim3((n_blocks + 255) / 256, rows), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), scores, ld, n_keys, block, out, n_blocks);
}

extern "C" int ds41_expand_blocks(const int* blocks, int rows, int k, int block, const int* limit, int* pos, int* count,
                                  void* stream) {
  if (blocks == nullptr || pos == nullptr || rows <= 0 || k <= 0 || block <= 0) return cudaErrorInvalidValue;
  return launch_pdl(expand_blocks_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), blocks, k, block,
                    limit, pos, count);
}
