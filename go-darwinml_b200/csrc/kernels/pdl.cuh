// Programmatic dependent launch: device-side hooks and the host-side launch helper.
//
// A kernel launched through launch_dependent() may start while the kernel before it on the stream is still running:
// everything up to pdl_wait() (barrier set-up, TMEM allocation, index arithmetic) then runs under that kernel's tail,
// and pdl_wait() returns once that kernel has completed and its writes are visible.  A kernel must not read or write
// global memory before its pdl_wait().  pdl_launch_dependents() lets the NEXT kernel's CTAs be scheduled as soon as
// every CTA of this one has called it (they still wait in their own pdl_wait()).  In a kernel launched the plain way
// both are no-ops, and a recorded plan keeps the relation as a programmatic edge between the two kernel nodes.
// B200MLX_PDL=0 launches everything the plain way.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace b200 {
namespace k {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool on = []() { const char* v = getenv("B200MLX_PDL"); return !(v && v[0] == '0'); }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = on ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The same with a grid and a block of up to three dimensions.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent_dims(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool on = []() { const char* v = getenv("B200MLX_PDL"); return !(v && v[0] == '0'); }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = on ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace k
}  // namespace b200
