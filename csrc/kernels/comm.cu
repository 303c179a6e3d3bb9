// Collective epilogues over NVLink peer memory.
//
//  rs_reduce : second half of the fused GEMM -> reduce-scatter.  Every source rank's GEMM epilogue stored its partial
//              rows for this rank into slot[src] of this rank's symmetric buffer; after a bounded wait on the peers'
//              epoch flags the slots are summed in rank order (deterministic) into bf16 or fp32 rows.
//              `as_bf16` bit 0: bf16 output; bit 1: the slots hold bf16 (TMA-store epilogue) instead of fp32.
//  The flags follow the library-wide protocol: a rank publishes "my stores for this step are complete" by raising its
//  epoch flag (ds41_signal); waiters spin with a cycle limit and report through the status word instead of hanging.
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

__global__ void __launch_bounds__(256)
rs_reduce_kernel(const float* __restrict__ slots, int world, long long slot_stride, void* __restrict__ out, int as_bf16,
                 long long n, const uint32_t* const* __restrict__ wait_flags, const uint32_t* __restrict__ wait_epoch,
                 int* status) {
  pdl_launch_dependents();
  pdl_wait();
  if (wait_flags != nullptr && world > 1) {
    if (threadIdx.x < world) flag_wait_ge(wait_flags[threadIdx.x], *wait_epoch, status, 600 + threadIdx.x);
    __syncthreads();
  }
  const long long i = (1ll * blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool slots_bf16 = (as_bf16 & 2) != 0;
  as_bf16 &= 1;
  for (int s = 0; s < world; ++s) {
    if (slots_bf16) {
      const uint2 q = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(slots) +
                                                            s * slot_stride + i));
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
      acc.x += lo.x; acc.y += lo.y; acc.z += hi.x; acc.w += hi.y;
    } else {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(slots + s * slot_stride + i));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  }
  if (as_bf16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + i) = o;
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(out) + i) = acc;
  }
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_rs_reduce(const float* slots, int world, long long slot_stride, void* out, int as_bf16,
                              long long n, const void* wait_flags, const void* wait_epoch, int* status, void* stream) {
  if (world <= 0 || world > 8 || n <= 0 || (n & 3)) return cudaErrorInvalidValue;
  const long long threads = n / 4;
  return launch_pdl(rs_reduce_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), slots, world, slot_stride, out, as_bf16, n,
                    reinterpret_cast<const uint32_t* const*>(wait_flags), reinterpret_cast<const uint32_t*>(wait_epoch),
                    status);
}
