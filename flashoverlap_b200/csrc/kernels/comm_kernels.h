// Small communication kernels over peer-mapped memory: the primitives the
// bandwidth tool times (peer-to-peer stores from registers, bulk stores from
// shared memory, NVLink SHARP load-reduce / multicast store / both) and a
// bounded counter wait.
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

// Same transfer with the bulk-copy engine: every warp stages `chunk_bytes`
// (multiple of 16, at most 16 KiB) of the source in shared memory with
// cp.async.bulk and sends it on with cp.async.bulk.global.shared::cta, three
// chunks in flight per warp.  No cluster multicast anywhere.
cudaError_t launch_p2p_push_bulk(const PushParams& p, int chunk_bytes, int ctas, cudaStream_t stream);

// NVLink SHARP primitives on a multicast mapping (`mc_*` are multicast
// addresses, the others ordinary local addresses; all 16-byte aligned):
//   MM_LD_REDUCE  local_dst[i] = sum over ranks of stage[i]      (multimem.ld_reduce, fp32 accumulate)
//   MM_ST         result[i] on every rank = local_src[i]          (multimem.st)
//   MM_ALLREDUCE  result[i] on every rank = sum over ranks stage[i]
// Each rank handles `bytes` bytes starting at byte offset `offset` (its share).
// When a CTA is done it bumps `arrive` on every rank (multimem.red).
enum MultimemKind : int { MM_LD_REDUCE = 0, MM_ST = 1, MM_ALLREDUCE = 2 };
struct MultimemParams {
  int kind;
  int bf16;
  const void* mc_stage;
  void* mc_result;
  const void* local_src;
  void* local_dst;
  long long offset;
  long long bytes;
  uint32_t* mc_arrive;  // may be null
};
cudaError_t launch_multimem(const MultimemParams& p, int ctas, cudaStream_t stream);

// Grid-wide bounded wait until *counter >= target, one thread (used by tests
// and by the bandwidth tool to close a push with a device-side barrier).
// status (and its host mirror, if not null) receive ST_TIMEOUT_FLAG on expiry.
cudaError_t launch_wait_counter(const uint32_t* counter, uint32_t target, unsigned long long timeout_ns,
                                StatusWord* status, StatusWord* mirror, int rank, cudaStream_t stream);

// Raises every counter[i] (i < n) to at least cseg[i] * mult: a stream-ordered
// release which guarantees that stream waits on those counters end even when
// the kernel that should have counted gave up.
cudaError_t launch_raise_counters(int* counter, const int* cseg, int mult, int n, cudaStream_t stream);

}  // namespace fo
