// Host-side launch interface of the fused sm_100a kernel (no PyTorch types).
#pragma once

#include <cuda_runtime.h>

#include "fused_params.h"

namespace fo {

enum DType : int { DT_F16 = 0, DT_BF16 = 1 };

// Tile configurations selectable through the reference's `Algo` index
// (reference: src/tiling/gemm_tiling.cuh:3-10 lists its six; these are the
// tcgen05 shapes used here).  BK is always 64.
// ctas == 2: the tile is computed by a pair of CTAs (tcgen05.mma.cta_group::2),
// 128 rows each.
struct TileConfig {
  int bm, bn, bk;
  int ctas;
};
constexpr int kNumAlgos = 5;
inline TileConfig algo_config(int algo) {
  static const TileConfig table[kNumAlgos] = {
      {128, 256, 64, 1}, {128, 128, 64, 1}, {128, 64, 64, 1}, {256, 256, 64, 2}, {256, 128, 64, 2}};
  return table[(algo < 0 || algo >= kNumAlgos) ? 0 : algo];
}

struct GemmOperands {
  const void* A;  // [M, K] row-major
  const void* B;  // [N, K] row-major
  int M, N, K;
  DType dtype;
  int algo;
  int sm_count;  // CTAs to launch (<= SMs of the device); 0 = all
};

// Fills p.tmA / p.tmB / shape fields from `g`, validates shapes, launches.
// Everything else in `p` must already be set by the caller.  Returns
// cudaSuccess or an error; *why (if not null) receives a static message.
cudaError_t launch_fused(const GemmOperands& g, FusedParams& p, cudaStream_t stream, const char** why);

// Number of SMs of the current device (cached per device).
int device_sm_count();

}  // namespace fo
