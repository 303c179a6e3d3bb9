// Host-side TMA tensor-map construction without linking libcuda: the driver entry point
// is resolved through the runtime (cudaGetDriverEntryPoint).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ds41 {

enum class TmaDtype : int { kBF16 = 0, kU8 = 1, kF32 = 2, kU4x16Align16 = 3, kU4x16Align8 = 4 };

// 3-D row-major view {batch, rows, cols}: cols contiguous, `row_stride_bytes` between rows and
// `batch_stride_bytes` between batches.  The box is {1, box_rows, box_cols}.  `swizzle128` selects
// the 128-byte shared-memory swizzle (box_cols * elem_size must then be 128 bytes).
// Returns cudaSuccess or an error; never throws.
cudaError_t make_tensor_map_3d(CUtensorMap* out, const void* base, TmaDtype dtype, uint64_t cols, uint64_t rows,
                               uint64_t batch, uint64_t row_stride_bytes, uint64_t batch_stride_bytes,
                               uint32_t box_cols, uint32_t box_rows, bool swizzle128);

int sm_count();
int last_tensor_map_result();   // CUresult of the most recent cuTensorMapEncodeTiled call (0 = success)

}  // namespace ds41
