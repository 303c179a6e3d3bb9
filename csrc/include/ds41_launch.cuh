// Kernel launch helper with programmatic dependent launch (PDL).
//
// Every kernel in this library starts with pdl_launch_dependents() (lets the next kernel in the stream begin
// its prologue early) and executes pdl_wait() before its first access to memory that an earlier kernel may
// write.  The wait returns only when the preceding grid has completed and flushed, so the chain stays
// correct wherever the trigger sits; because every grid waits before it can complete, ordering is transitive.
// DS41_PDL=0 in the environment turns the launch attribute off (the device instructions are then no-ops).
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include <utility>

namespace ds41 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = std::getenv("DS41_PDL");
    cached = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace ds41
