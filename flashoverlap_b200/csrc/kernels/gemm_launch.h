// Host-side launch interface of the fused sm_100a kernel (no PyTorch types).
#pragma once

#include <cuda_runtime.h>

#include "fused_params.h"

namespace fo {

enum DType : int { DT_F16 = 0, DT_BF16 = 1 };

// Tile configurations selectable through the reference's `Algo` index
// (reference: src/tiling/gemm_tiling.cuh:3-10 lists its six).  The table, the
// per-instance source files and configs/AlgoDict.pt are written by
// tool/generate_instances.py, as in the reference (tool/generate_instances.py:5-63).
// ctas == 2: the tile is computed by a pair of CTAs (tcgen05.mma.cta_group::2),
// 128 rows each.
struct TileConfig {
  int bm, bn, bk;
  int ctas;
};
#include "generated/algo_count.inc"  // constexpr int kNumAlgos = ...;
TileConfig algo_config(int algo);

struct GemmOperands {
  const void* A;  // [M, K] row-major
  const void* B;  // [N, K] row-major
  int M, N, K;
  DType dtype;
  int algo;
  int sm_count;  // CTAs to launch (<= SMs of the device); 0 = all
  // Optional: rows [own_begin, own_begin + own_rows) of A are read from A_own
  // ([own_rows, K] row-major, 16-byte aligned) instead of from A.
  const void* A_own;
  int own_begin, own_rows;
};

// Fills p.tmA / p.tmB / shape fields from `g`, validates shapes, launches.
// Everything else in `p` must already be set by the caller.  Returns
// cudaSuccess or an error; *why (if not null) receives a static message.
cudaError_t launch_fused(const GemmOperands& g, FusedParams& p, cudaStream_t stream, const char** why);

// One-time set-up of an instance on the current device (its shared-memory
// limit), so that a later launch_fused enqueues work only.
cudaError_t prepare_fused(int algo, DType dtype);

// Number of SMs of the current device (cached per device).
int device_sm_count();

// Per-device caches (kernel attributes, SM counts) hold this many devices;
// a device with a higher index is handled uncached.
constexpr int kMaxDevices = 64;

// FLASHOVERLAP_COOPERATIVE=1 in the environment makes fused launches
// cooperative: the driver then guarantees that all CTAs are resident together
// (or refuses the launch), which matters when something else may hold SMs.
// Off by default: a profiler that replays kernels refused the cooperative
// launch (LaunchFailed under `ncu --set full`).  Without it, fused launches on
// one GPU must not overlap one another; a CTA that cannot become resident
// makes the waits of the resident ones run into their deadline.
bool cooperative_launch_enabled();

}  // namespace fo
