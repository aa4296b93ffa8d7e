#include "comm_kernels.h"

#include "gemm_fused_sm100.cuh"
#include "gemm_launch.h"

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

// One lane per warp drives a ring of kBulkBufs shared-memory buffers: bulk
// load of chunk i+1 from local memory while the bulk stores of chunks i,
// i-1, ... travel to the peer.  Work item = (destination, chunk).
constexpr int kBulkBufs = 3;
constexpr int kBulkWarps = 4;
__global__ void __launch_bounds__(kBulkWarps * 32) p2p_push_bulk_kernel(const PushParams p, int chunk_bytes) {
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ __align__(8) uint64_t bars[kBulkWarps * kBulkBufs];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kBulkWarps * kBulkBufs; ++i) ptx::mbar_init(&bars[i], 1);
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();
  const uint64_t deadline = ptx::globaltimer_ns() + 2000000000ull;
  if (lane == 0) {
    const int ndst = p.include_self ? p.ws : p.ws - 1;
    const long long per_dst = (p.bytes + chunk_bytes - 1) / chunk_bytes;
    const long long items = per_dst * ndst;
    const long long w = static_cast<long long>(blockIdx.x) * kBulkWarps + warp;
    const long long nw = static_cast<long long>(gridDim.x) * kBulkWarps;
    const uint32_t buf0 = ptx::smem_u32(bulk_smem) + static_cast<uint32_t>(warp * kBulkBufs * chunk_bytes);
    uint64_t* bar = bars + warp * kBulkBufs;
    const char* src = static_cast<const char*>(p.src);
    auto locate = [&](long long it, int& d, long long& off, uint32_t& n) {
      // destinations interleaved chunk by chunk
      const int r = static_cast<int>(it % ndst);
      const long long c = it / ndst;
      d = p.me + 1 + r;
      if (d >= p.ws) d -= p.ws;
      off = c * chunk_bytes;
      const long long left = p.bytes - off;
      n = static_cast<uint32_t>(left < chunk_bytes ? left : chunk_bytes);
    };
    bool ok = true;
    int k = 0;  // items issued by this warp
    uint32_t phases = 0;
    int d;
    long long off;
    uint32_t n;
    if (w < items) {
      locate(w, d, off, n);
      ptx::mbar_arrive_expect_tx(&bar[0], n);
      ptx::bulk_load_1d(buf0, src + d * p.src_stride + off, n, &bar[0]);
    }
    for (long long it = w; it < items && ok; it += nw, ++k) {
      const int b = k % kBulkBufs;
      locate(it, d, off, n);
      if (it + nw < items) {
        // the buffer of item k+1 was last read by the store of item k+1-kBulkBufs
        ptx::bulk_wait_group_read<kBulkBufs - 2>();
        int d2;
        long long off2;
        uint32_t n2;
        locate(it + nw, d2, off2, n2);
        const int b2 = (k + 1) % kBulkBufs;
        ptx::mbar_arrive_expect_tx(&bar[b2], n2);
        ptx::bulk_load_1d(buf0 + static_cast<uint32_t>(b2 * chunk_bytes), src + d2 * p.src_stride + off2, n2, &bar[b2]);
      }
      if (!ptx::mbar_wait(&bar[b], (phases >> b) & 1u, deadline)) {
        ok = false;
        break;
      }
      phases ^= 1u << b;
      ptx::bulk_store_1d(static_cast<char*>(p.dst[d]) + off, buf0 + static_cast<uint32_t>(b * chunk_bytes), n);
      ptx::bulk_commit_group();
    }
    ptx::bulk_wait_group<0>();   // all stores of this warp are complete
    ptx::fence_proxy_async_all();  // async-proxy writes before the generic-proxy release below
  }
  __syncthreads();
  if (p.flag[0] != nullptr && threadIdx.x < p.ws) {
    const int dd = threadIdx.x;
    if ((dd != p.me || p.include_self) && p.flag[dd] != nullptr) ptx::red_release_sys_add(p.flag[dd], 1u);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256) multimem_kernel(const MultimemParams p) {
  constexpr int U = 8;
  const long long chunks = p.bytes >> 4;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const char* stage = static_cast<const char*>(p.mc_stage) + p.offset;
  char* result = static_cast<char*>(p.mc_result) + p.offset;
  const char* lsrc = static_cast<const char*>(p.local_src) + p.offset;
  char* ldst = static_cast<char*>(p.local_dst) + p.offset;
  for (long long c0 = tid; c0 < chunks; c0 += nthreads * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long c = c0 + u * nthreads;
      if (c < chunks) {
        if (p.kind == MM_ST) v[u] = *reinterpret_cast<const uint4*>(lsrc + (c << 4));
        else v[u] = ptx::multimem_ld_reduce_add_v4<BF16>(stage + (c << 4));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long c = c0 + u * nthreads;
      if (c < chunks) {
        if (p.kind == MM_LD_REDUCE) ptx::st_v4(ldst + (c << 4), v[u]);
        else ptx::multimem_st_v4(result + (c << 4), v[u]);
      }
    }
  }
  if (p.mc_arrive != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      ptx::fence_acq_rel_sys();
      ptx::multimem_red_release_add(p.mc_arrive, 1u);
    }
  }
}

__global__ void wait_counter_kernel(const uint32_t* counter, uint32_t target, unsigned long long timeout_ns,
                                    StatusWord* status, StatusWord* mirror, int rank) {
  const uint64_t deadline = ptx::globaltimer_ns() + timeout_ns;
  uint32_t seen = 0;
  if (!ptx::wait_counter_geq(counter, target, deadline, &seen)) {
    report_error(status, mirror, ST_TIMEOUT_FLAG, rank, 0xF00u, seen, target);
  }
}

__global__ void raise_counters_kernel(int* counter, const int* cseg, int mult, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicMax(counter + i, cseg[i] * mult);
}

}  // namespace

cudaError_t launch_p2p_push(const PushParams& p, int ctas, cudaStream_t stream) {
  if (p.bytes < 0 || (p.bytes & 15) != 0 || p.ws < 1 || p.ws > kMaxRanks) return cudaErrorInvalidValue;
  if (ctas <= 0) ctas = device_sm_count();
  p2p_push_kernel<<<ctas, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_p2p_push_bulk(const PushParams& p, int chunk_bytes, int ctas, cudaStream_t stream) {
  if (p.bytes < 0 || (p.bytes & 15) != 0 || p.ws < 1 || p.ws > kMaxRanks) return cudaErrorInvalidValue;
  if (chunk_bytes < 16 || chunk_bytes > 16384 || (chunk_bytes & 15) != 0) return cudaErrorInvalidValue;
  if (ctas <= 0) ctas = device_sm_count();
  const int smem = kBulkWarps * kBulkBufs * chunk_bytes;
  static bool attr_set[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < kMaxDevices && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(p2p_push_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kBulkWarps * kBulkBufs * 16384);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  p2p_push_bulk_kernel<<<ctas, kBulkWarps * 32, smem, stream>>>(p, chunk_bytes);
  return cudaGetLastError();
}

cudaError_t launch_multimem(const MultimemParams& p, int ctas, cudaStream_t stream) {
  if (p.bytes < 0 || (p.bytes & 15) != 0 || (p.offset & 15) != 0) return cudaErrorInvalidValue;
  if (ctas <= 0) ctas = device_sm_count();
  if (p.bf16) multimem_kernel<true><<<ctas, 256, 0, stream>>>(p);
  else multimem_kernel<false><<<ctas, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_wait_counter(const uint32_t* counter, uint32_t target, unsigned long long timeout_ns,
                                StatusWord* status, StatusWord* mirror, int rank, cudaStream_t stream) {
  wait_counter_kernel<<<1, 1, 0, stream>>>(counter, target, timeout_ns, status, mirror, rank);
  return cudaGetLastError();
}

cudaError_t launch_raise_counters(int* counter, const int* cseg, int mult, int n, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  raise_counters_kernel<<<1, 128, 0, stream>>>(counter, cseg, mult, n);
  return cudaGetLastError();
}

}  // namespace fo
