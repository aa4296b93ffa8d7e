// Small communication kernels over peer-mapped memory: the primitives the
// bandwidth tool times and the all-gather push used in front of a GEMM.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "fused_params.h"

namespace fo {

struct PushParams {
  const void* src;           // local source
  void* dst[kMaxRanks];      // destination on each rank (entry `me` may be local or null)
  uint32_t* flag[kMaxRanks]; // optional: counter on each destination, +1 per CTA when its share is written
  long long bytes;           // bytes sent to EACH destination (multiple of 16)
  long long src_stride;      // distance between the source blocks for successive destinations (0 = same block)
  int ws, me;
  int include_self;
};

// Every rank copies `bytes` from src (+ r * src_stride for destination r) to
// dst[r] for all r != me (and r == me when include_self) with 16-byte stores,
// destinations interleaved chunk by chunk so that all links are busy at once.
cudaError_t launch_p2p_push(const PushParams& p, int ctas, cudaStream_t stream);

// Grid-wide bounded wait until *counter >= target, one thread (used by tests
// and by the bandwidth tool to close a push with a device-side barrier).
// status receives ST_TIMEOUT_FLAG on expiry.
cudaError_t launch_wait_counter(const uint32_t* counter, uint32_t target, unsigned long long timeout_ns,
                                StatusWord* status, int rank, cudaStream_t stream);

}  // namespace fo
