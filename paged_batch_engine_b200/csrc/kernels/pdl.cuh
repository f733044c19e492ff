// Programmatic dependent launch: a kernel launched with this attribute may start while
// the kernel before it in the stream is still draining.  Its blocks run up to
// pdl_wait(), which returns once the previous kernel has completed and its writes are
// visible; everything a kernel reads from or writes to activations, the cache or any
// other buffer of the step comes after that call.  What does not depend on the previous
// kernel (weights, above all) may be fetched before it.  pdl_launch_dependents() tells
// the next kernel it may begin launching: the weight-streaming kernels call it where their
// blocks have issued most of their memory traffic, the short kernels between them (norms,
// position encoding, merge, activation, sampling) at their very top, before their own
// wait, so that the next weight-streaming kernel is resident and fetching while they run.
// Inside a captured graph the same launches become programmatic dependency edges.  Every block of every kernel calls pdl_wait() before it
// exits, so "the previous kernel completed" always implies that all earlier ones did.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace pbe {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("PBE_PDL");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args... args) {
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
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with a thread-block cluster of `cluster` blocks along x (1: no cluster).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, int cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace pbe
