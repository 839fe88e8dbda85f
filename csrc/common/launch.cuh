// Kernel launch with programmatic dependent launch (PDL).
//
// Kernels on the decode path are launched with programmaticStreamSerialization: the next kernel's
// CTAs become resident while the previous kernel drains, and block in griddep_wait() until the
// previous grid has completed and flushed.  Every such kernel executes griddep_wait() before its
// first dependent read and before its first global write (and before any early return), which
// keeps the stream's ordering guarantees intact; griddep_launch() lets the NEXT kernel start early.
// On a launch without the attribute both instructions are no-ops.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace b200 {

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Process-wide switch (default on; B200_PDL=0 in the environment turns it off).
int pdl_enabled();
int gemm_l2_prefetch();
// Raises a kernel's dynamic shared-memory limit to at least `bytes` on the CURRENT device, once per
// (kernel, device) pair: the attribute belongs to the device context, so a process that drives several GPUs must
// set it on each of them (defined in runtime/tma.cpp).
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

// Same, with a thread-block cluster of `cluster` CTAs (cluster.x * cluster.y * cluster.z <= 8; grid divisible by it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                      cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster.x;
  attr[1].val.clusterDim.y = cluster.y;
  attr[1].val.clusterDim.z = cluster.z;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

}  // namespace b200
