// Host-side kernel launch helper shared by every translation unit of the library.
//
// Kernels of a serving step are short (10-70 us), so what happens BETWEEN two kernels counts: the launch latency,
// the set-up of the next kernel (barrier initialisation, tensor-memory allocation, tensor-map prefetch, the first
// weight copies) and the tail of the previous one, during which most SMs idle.  Programmatic dependent launch
// overlaps them: a kernel launched through `launch()` may start while its predecessor in the stream is still
// running, as soon as every CTA of the predecessor has executed `pdl_launch_dependents()` (or exited); it runs its
// own set-up, then blocks in `pdl_wait()` until the predecessor has completed and its memory is visible.
//
// Rules every kernel launched here follows:
//   * it calls pdl_wait() before its first access to global memory that another kernel writes, and before its
//     first global write (an earlier kernel may still be reading the destination);
//   * before pdl_wait() it touches only shared / tensor memory and operands that no kernel writes (the weights);
//   * pdl_launch_dependents() comes after pdl_wait(), so completion stays transitive along the stream.
// A kernel launched without the attribute (PyTorch's own, or with the switch off) orders itself after the
// whole predecessor as usual; pdl_wait() then returns at once.  The attribute is captured into CUDA graphs
// as a programmatic dependency edge.
#pragma once
#include <cuda_runtime.h>

extern "C" int cb_pdl_enabled();

namespace cb {

template <typename... KArgs, typename... Args>
static inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  if (cb_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  return launch(kernel, grid, block, smem, stream, dim3(1, 1, 1), args...);
}

}  // namespace cb
