// Programmatic dependent launch for chains of short kernels (the decode step).
//
// A decode step is a few hundred dependent kernels of a few microseconds each; between two of them the GPU idles
// for the launch latency and the next kernel's prologue (barrier set-up, first weight loads). A kernel launched
// through `launch_pdl` may be scheduled as soon as every CTA of its predecessor has executed `pdl_launch_dependents()`
// (or exited): it then runs whatever does not depend on the predecessor (here: prefetching its weights, which no
// kernel writes) and calls `pdl_wait()`, which returns once the predecessor has completed and its writes are
// visible. Rules every kernel launched this way follows:
//   * before `pdl_wait()` it reads only memory no kernel of the chain writes (weights) and writes nothing global;
//   * a kernel launched the ordinary way still waits for the full completion of what precedes it, and an ordinary
//     predecessor releases its dependent when it exits, so the two kinds mix freely on one stream;
//   * both calls are no-ops in a kernel that was launched the ordinary way.
// `MILES_B200_PDL=0` in the environment turns the attribute off (every launch becomes an ordinary one).
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace mb {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("MILES_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

}  // namespace mb
