// Tensor-map construction and small device queries shared by the tensor-core kernels.
#include "ds41_tma.h"

#include <mutex>

namespace ds41 {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;

void resolve() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<EncodeFn>(fn);
  }
}
}  // namespace

static int g_last_result = 0;     // driver result of the most recent encode (diagnostics)

cudaError_t make_tensor_map_3d(CUtensorMap* out, const void* base, TmaDtype dtype, uint64_t cols, uint64_t rows,
                               uint64_t batch, uint64_t row_stride_bytes, uint64_t batch_stride_bytes,
                               uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
  std::call_once(g_once, resolve);
  if (g_encode == nullptr) return cudaErrorNotSupported;
  CUtensorMapDataType dt;
  uint32_t elem_bits;
  switch (dtype) {
    case TmaDtype::kBF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; elem_bits = 16; break;
    case TmaDtype::kU8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; elem_bits = 8; break;
    case TmaDtype::kF32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; elem_bits = 32; break;
    case TmaDtype::kU4x16Align16: dt = CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B; elem_bits = 4; break;
    case TmaDtype::kU4x16Align8: dt = CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B; elem_bits = 4; break;   // packed in smem too
    default: return cudaErrorInvalidValue;
  }
  // 4-bit elements packed two per byte in global memory land one per byte in shared memory (16 values per 16 bytes):
  // the box must be 128 elements wide and addresses / strides need 32-byte alignment
  const bool padded4 = dtype == TmaDtype::kU4x16Align16;
  const uint64_t box_smem_bytes = padded4 ? box_cols : uint64_t(box_cols) * elem_bits / 8;
  const uint64_t align = padded4 ? 31 : 15;
  if ((reinterpret_cast<uintptr_t>(base) & align) != 0 || (row_stride_bytes & align) != 0 ||
      (batch > 1 && (batch_stride_bytes & align) != 0) || (box_smem_bytes & 15) != 0 ||
      box_rows == 0 || box_rows > 256 || box_cols == 0 || box_cols > 256 || (padded4 && (box_cols != 128 || cols % 128))) {
    return cudaErrorInvalidValue;
  }
  if (swizzle128 && box_smem_bytes != 128) return cudaErrorInvalidValue;
  cuuint64_t dims[3] = {cols, rows, batch == 0 ? 1 : batch};
  cuuint64_t strides[2] = {row_stride_bytes, batch > 1 ? batch_stride_bytes : row_stride_bytes * rows};
  if ((strides[1] & align) != 0) strides[1] = (strides[1] + align) & ~align;
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_result = static_cast<int>(r);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

int last_tensor_map_result() { return g_last_result; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace ds41
