// One template instance of the fused kernel and its launcher.  Every generated
// file under generated/ includes this header and defines one launcher with
// FO_DEFINE_GEMM_INSTANCE, so that the instances compile in parallel.
#pragma once

#include <cuda_runtime.h>

#include "gemm_fused_sm100.cuh"
#include "gemm_launch.h"

namespace fo {

// Launches one CTA per requested SM (a cluster of two for CTA pairs), as a
// cooperative launch when cooperative_launch_enabled().
// Raises the kernel's dynamic shared-memory limit on the current device (once
// per device and instance; a device index beyond the cache is set every time).
template <int BN, int BK, bool BF16, int CTAS>
cudaError_t prepare_instance() {
  using T = TileTraits<BN, CTAS, BK>;
  static bool attr_set[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices || !attr_set[dev]) {
    e = cudaFuncSetAttribute(gemm_fused_sm100_kernel<BN, BK, BF16, CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             T::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < kMaxDevices) attr_set[dev] = true;
  }
  return cudaSuccess;
}

template <int BN, int BK, bool BF16, int CTAS>
cudaError_t launch_instance(const FusedParams& p, int grid, cudaStream_t stream) {
  using T = TileTraits<BN, CTAS, BK>;
  auto kern = gemm_fused_sm100_kernel<BN, BK, BF16, CTAS>;
  cudaError_t e = prepare_instance<BN, BK, BF16, CTAS>();
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(CTAS == 2 ? (grid & ~1) : grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (CTAS == 2) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 2;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (cooperative_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeCooperative;
    attr[n].val.cooperative = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace fo

#define FO_DEFINE_GEMM_INSTANCE(NAME, BN, BK, BF16, CTAS)                                    \
  namespace fo {                                                                             \
  cudaError_t NAME(const FusedParams& p, int grid, cudaStream_t stream) {                    \
    return launch_instance<BN, BK, BF16, CTAS>(p, grid, stream);                             \
  }                                                                                          \
  cudaError_t NAME##_prepare() { return prepare_instance<BN, BK, BF16, CTAS>(); }            \
  }
