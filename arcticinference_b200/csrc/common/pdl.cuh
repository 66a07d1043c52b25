// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may
// start while the kernel before it in the stream is still running. Its threads run up to
// `pdl_wait()`, which returns once every earlier kernel of the stream has finished and its
// writes are visible; what comes before the wait (barrier and TMEM set-up, tensor-map
// prefetch, loads of weights that no kernel writes) overlaps the earlier kernel's tail, and
// the launch latency disappears behind it. `pdl_trigger()` tells the scheduler that the next
// kernel of the stream may be placed; it is issued as early as possible because the next
// kernel protects itself with its own wait.
//
// Rules every kernel launched through `launch_pdl` follows:
//   * no global write and no read of data another kernel produces before `pdl_wait()`;
//   * every thread that touches such data executes `pdl_wait()` first.
// A kernel launched without the attribute sees both instructions as no-ops, and a kernel
// launched with a plain <<<>>> after one of these waits for its full completion as usual.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace ab200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Off unless AB200_PDL=1: measured end to end, the overlap gains 2 us per back-to-back decode
// GEMM in isolation and loses about 1 % on the serving benchmark (on one and on two GPUs),
// whose decode steps are replayed from CUDA graphs and whose early-resident successor CTAs
// compete with the running kernel for the memory system. Without the attribute the two
// griddepcontrol instructions are no-ops and kernels follow ordinary stream order.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("AB200_PDL");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

// `cluster_x` > 1 launches thread-block clusters of that many consecutive blocks (grid.x must
// be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                      size_t smem, cudaStream_t stream, unsigned cluster_x,
                                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster_x > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  return launch_pdl_cluster(kernel, grid, block, smem, stream, 1u, std::forward<Args>(args)...);
}

}  // namespace ab200
