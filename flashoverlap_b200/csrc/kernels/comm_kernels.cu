#include "comm_kernels.h"

#include "gemm_fused_sm100.cuh"

namespace fo {

namespace {

__global__ void __launch_bounds__(256) p2p_push_kernel(const PushParams p) {
  const long long chunks = p.bytes >> 4;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const char* src = static_cast<const char*>(p.src);
  for (long long c = tid; c < chunks; c += nthreads) {
#pragma unroll 1
    for (int r = 0; r < p.ws; ++r) {
      int d = p.me + 1 + r;
      if (d >= p.ws) d -= p.ws;
      if (d == p.me && !p.include_self) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(src + d * p.src_stride + (c << 4));
      ptx::st_v4(static_cast<char*>(p.dst[d]) + (c << 4), v);
    }
  }
  if (p.flag[0] != nullptr) {
    __syncthreads();
    if (threadIdx.x < p.ws) {
      const int d = threadIdx.x;
      if ((d != p.me || p.include_self) && p.flag[d] != nullptr) ptx::red_release_sys_add(p.flag[d], 1u);
    }
  }
}

__global__ void wait_counter_kernel(const uint32_t* counter, uint32_t target, unsigned long long timeout_ns,
                                    StatusWord* status, int rank) {
  const uint64_t deadline = ptx::globaltimer_ns() + timeout_ns;
  uint32_t seen = 0;
  if (!ptx::wait_counter_geq(counter, target, deadline, &seen)) {
    report_error(status, ST_TIMEOUT_FLAG, rank, 0xF00u, seen, target);
  }
}

}  // namespace

cudaError_t launch_p2p_push(const PushParams& p, int ctas, cudaStream_t stream) {
  if (p.bytes < 0 || (p.bytes & 15) != 0 || p.ws < 1 || p.ws > kMaxRanks) return cudaErrorInvalidValue;
  if (ctas <= 0) ctas = 148;
  p2p_push_kernel<<<ctas, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_wait_counter(const uint32_t* counter, uint32_t target, unsigned long long timeout_ns,
                                StatusWord* status, int rank, cudaStream_t stream) {
  wait_counter_kernel<<<1, 1, 0, stream>>>(counter, target, timeout_ns, status, rank);
  return cudaGetLastError();
}

}  // namespace fo
