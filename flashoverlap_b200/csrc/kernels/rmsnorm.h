// Stand-alone RMSNorm kernels (no PyTorch types).
#pragma once

#include <cuda_runtime.h>

#include "fused_params.h"
#include "gemm_launch.h"

namespace fo {

// out[r][:] = round16(x[r][:] * rsqrt(mean(x[r][:]^2) + eps)) * w[:], natural
// layout in and out.  dim % 8 == 0.
cudaError_t launch_rmsnorm(const void* x, void* out, const void* w, int rows, int dim, float eps, DType dt,
                           cudaStream_t stream);

// Same, but x is stored in the tile-reordered layout described by `in_layout`
// (OutLayout::tiled == 1) and the output is written in natural order.
cudaError_t launch_reorder_rmsnorm(const void* x, void* out, const void* w, int rows, int dim, float eps,
                                   const OutLayout& in_layout, DType dt, cudaStream_t stream);

}  // namespace fo
