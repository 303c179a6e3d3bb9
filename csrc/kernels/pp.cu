// Pipeline-stage handoff over peer memory: the producer stage copies its boundary state into its own symmetric slot and
// raises a counter; the consumer stage's kernel waits (bounded) for that counter through a peer pointer and pulls the
// slot with plain 16-byte peer loads.  A second counter travelling the other way tells the producer that a slot was
// consumed, so two slots are enough to let the stages overlap.
//   pp_signal : publish `value` in this rank's counter after all earlier work of the stream (release at system scope)
//   pp_wait   : wait until a (peer) counter reaches `value`
//   pp_pull   : wait, then copy `nbytes` from a (peer) buffer into local memory
// Design parity: the residual handoff between the two layer stages of the reference's dual-GPU mode
// (rust/crates/ds41rt-daemon/src/v41_block/transfer.rs, native/cuda/kernels/v41_peer_copy.cu:6-80).
#include "ds41_api.h"
#include "ds41_launch.cuh"
#include "ds41_ptx.cuh"

namespace ds41 {

__global__ void pp_signal_kernel(uint32_t* flag, uint32_t value) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
  }
}

__global__ void pp_wait_kernel(const uint32_t* flag, uint32_t value, int* status, int site) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) flag_wait_ge(flag, value, status, site);
}

__global__ void __launch_bounds__(256)
pp_pull_kernel(const uint4* src, uint4* dst, long long n16, const uint32_t* flag, uint32_t value, int* status,
               int site) {
  __shared__ int ok;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) ok = flag_wait_ge(flag, value, status, site) ? 1 : 0;
  __syncthreads();
  if (!ok) return;                                   // the status word names the site; nothing is copied
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += 1ll * gridDim.x * blockDim.x)
    dst[i] = __ldcg(src + i);
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_pp_signal(void* flag, unsigned value, void* stream) {
  if (flag == nullptr) return cudaErrorInvalidValue;
  return launch_pdl(pp_signal_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                    static_cast<uint32_t*>(flag), value);
}

extern "C" int ds41_pp_wait(const void* flag, unsigned value, int* status, int site, void* stream) {
  if (flag == nullptr) return cudaErrorInvalidValue;
  return launch_pdl(pp_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint32_t*>(flag), value, status, site);
}

extern "C" int ds41_pp_pull(const void* src, void* dst, long long nbytes, const void* flag, unsigned value,
                            int* status, int site, void* stream) {
  if (src == nullptr || dst == nullptr || flag == nullptr || nbytes <= 0 || (nbytes & 15)) return cudaErrorInvalidValue;
  const long long n16 = nbytes / 16;
  int blocks = static_cast<int>((n16 + 255) / 256);
  if (blocks > 148) blocks = 148;
  return launch_pdl(pp_pull_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint4*>(src), static_cast<uint4*>(dst), n16, static_cast<const uint32_t*>(flag),
                    value, status, site);
}
