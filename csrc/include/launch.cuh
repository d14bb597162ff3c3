// One way to launch every kernel of the library: cudaLaunchKernelEx with
//   * programmatic dependent launch (PDL): the kernel may start while its predecessor in the stream is still
//     running; it executes `griddepcontrol.wait` (pdl_wait) before touching anything the predecessor produces.
//     Every kernel calls pdl_wait exactly once on every path, so completion stays transitive along the stream.
//     What a kernel does BEFORE pdl_wait overlaps with the predecessor's tail: barrier and tensor-memory set-up,
//     tensor-map prefetch and, in the decode GEMM, the first weight tiles (weights never depend on a predecessor).
//   * an optional thread-block cluster dimension along y (cluster_y >= 1; 0 = not a cluster kernel).  A kernel
//     that executes cluster instructions (barrier.cluster, mapa, shared::cluster bulk copies) is ALWAYS launched
//     with the attribute, also for a cluster of one CTA: launched without it, the decode GEMM raised
//     "illegal instruction" on B200.
// CUDA-graph capture records these launches with programmatic edges.  FORGE_PDL=0 in the environment switches
// the attribute off (kernels then see griddepcontrol.* as no-ops).
#pragma once

#include <atomic>
#include <cuda_runtime.h>

#include <cstdlib>

namespace forge {

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("FORGE_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// The dynamic shared memory limit of a kernel is a per-DEVICE attribute: raise it once per (call site, device), so a
// process that drives several GPUs gets it on each of them.  Used inside launchers that return an int code (-4 on failure).
#define FORGE_ENSURE_DYN_SMEM(kern, bytes)                                                                              \
  do {                                                                                                                  \
    static bool forge_attr_set[64] = {};                                                                                \
    int forge_dev = 0;                                                                                                  \
    if (cudaGetDevice(&forge_dev) != cudaSuccess || forge_dev < 0 || forge_dev >= 64) return -4;                        \
    if (!forge_attr_set[forge_dev]) {                                                                                   \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -4;     \
      forge_attr_set[forge_dev] = true;                                                                                 \
    }                                                                                                                   \
  } while (0)

// Streaming multiprocessors of the current device (queried once per device; grid and tile heuristics are stated in
// multiples of it instead of a fixed 148).
inline int device_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Kernels of this library launched (or captured into a CUDA graph) by this process so far: what the benchmark reports as
// its launch count.  One counter for the whole shared object.
inline std::atomic<long long>& launch_counter() {
  static std::atomic<long long> n{0};
  return n;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 int cluster_y, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_y >= 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = static_cast<unsigned>(cluster_y);
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e == cudaSuccess) launch_counter().fetch_add(1, std::memory_order_relaxed);
  return e;
}

// The same with clusters of `cluster_x` CTAs along x (CTA pairs of the cta_group::2 kernels: ranks 2i, 2i + 1 = blockIdx.x).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                           int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
  attr[n].val.clusterDim.y = 1;
  attr[n].val.clusterDim.z = 1;
  ++n;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e == cudaSuccess) launch_counter().fetch_add(1, std::memory_order_relaxed);
  return e;
}

}  // namespace forge
