// Allocation-free GEMM + RMSNorm entry point; see no_alloc_entry.h for the
// contract.  The scratch memory of the fused kernel (the un-normalised product
// and the per-tile-row arrival counters) lives in a file-scope device array.
#include "no_alloc_entry.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "fused_params.h"
#include "gemm_launch.h"

namespace {

using fo::kFlagWords;
using fo::kMaxDevices;
using fo::kMaxTileRows;                                  // arrival counters, one per 128 rows
constexpr size_t kCounterBytes = 16 * 1024;              // >= kFlagWords * 4, keeps the product 256-byte aligned
constexpr size_t kProductBytes = static_cast<size_t>(FO_NOALLOC_MAX_ELEMS) * 2;
static_assert(kCounterBytes >= static_cast<size_t>(kFlagWords) * 4, "counter area too small");

// [counters | product].  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address is looked up once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kCounterBytes + kProductBytes];

struct DeviceSlot {
  std::once_flag once;
  void* scratch = nullptr;
  cudaError_t error = cudaSuccess;
};
DeviceSlot g_slots[kMaxDevices];

int fail(int code, char* err, size_t err_len, const char* msg) {
  if (err != nullptr && err_len > 0) {
    std::snprintf(err, err_len, "%s", msg);
  }
  return code;
}

}  // namespace

extern "C" int fo_gemm_rmsnorm_noalloc(const void* A, const void* B, const void* gamma, void* out, int M, int N,
                                       int K, int dtype, float eps, void* stream, void* status32, char* err,
                                       size_t err_len) {
  if (A == nullptr || B == nullptr || gamma == nullptr || out == nullptr) {
    return fail(1, err, err_len, "fo_gemm_rmsnorm_noalloc: A, B, gamma and out must not be null");
  }
  if (dtype != 0 && dtype != 1) return fail(1, err, err_len, "fo_gemm_rmsnorm_noalloc: dtype must be 0 (fp16) or 1 (bf16)");
  if (M <= 0 || N <= 0 || K <= 0 || M % 128 != 0 || N % 256 != 0 || K % 8 != 0) {
    return fail(2, err, err_len, "fo_gemm_rmsnorm_noalloc: need M % 128 == 0, N % 256 == 0, K % 8 == 0");
  }
  if (static_cast<long long>(M) * N > FO_NOALLOC_MAX_ELEMS || M / 128 > kMaxTileRows) {
    char msg[200];
    std::snprintf(msg, sizeof(msg),
                  "fo_gemm_rmsnorm_noalloc: M*N = %lld exceeds the built-in scratch of %lld values (or M > %d)",
                  static_cast<long long>(M) * N, static_cast<long long>(FO_NOALLOC_MAX_ELEMS), 128 * kMaxTileRows);
    return fail(3, err, err_len, msg);
  }
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u) ||
      (reinterpret_cast<uintptr_t>(gamma) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) {
    return fail(1, err, err_len, "fo_gemm_rmsnorm_noalloc: A, B, gamma and out must be 16-byte aligned");
  }

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(4, err, err_len, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(4, err, err_len, "fo_gemm_rmsnorm_noalloc: device index out of range");

  // Set-up, once per device, with that device current: the device address of
  // the scratch array (the host-side symbol is not usable as a pointer) and the
  // shared-memory limit of the kernel for both dtypes.
  DeviceSlot& slot = g_slots[dev];
  std::call_once(slot.once, [&slot] {
    void* ptr = nullptr;
    slot.error = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (slot.error == cudaSuccess) slot.scratch = ptr;
    if (slot.error == cudaSuccess) slot.error = fo::prepare_fused(0, fo::DT_F16);
    if (slot.error == cudaSuccess) slot.error = fo::prepare_fused(0, fo::DT_BF16);
  });
  if (slot.error != cudaSuccess || slot.scratch == nullptr) {
    return fail(5, err, err_len, "fo_gemm_rmsnorm_noalloc: set-up failed (cudaGetSymbolAddress / shared-memory limit)");
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned char* base = static_cast<unsigned char*>(slot.scratch);
  uint32_t* counters = reinterpret_cast<uint32_t*>(base);
  void* product = base + kCounterBytes;

  // The counters keep the previous call's values: clear them.
  e = cudaMemsetAsync(counters, 0, static_cast<size_t>(kFlagWords) * sizeof(uint32_t), s);
  if (e != cudaSuccess) return fail(6, err, err_len, cudaGetErrorString(e));

  fo::GemmOperands g{};
  g.A = A;
  g.B = B;
  g.M = M;
  g.N = N;
  g.K = K;
  g.dtype = dtype == 1 ? fo::DT_BF16 : fo::DT_F16;
  g.algo = 0;  // 128 x 256 tiles, one CTA per tile
  g.sm_count = 0;

  fo::FusedParams p{};
  p.own_mode = fo::OWN_SINGLE;
  p.ws = 1;
  p.me = 0;
  p.rows_per_owner = M;
  p.epi_base[0] = product;
  p.epi_layout.ld = N;
  p.flag[0] = counters;
  p.job_counter = counters + fo::kFlagJob;
  p.raster_group = 4;
  p.reduce = 1;
  p.stage = product;
  p.flag_target = static_cast<uint32_t>(N / 256);  // one arrival per tile of the 128-row block
  p.norm = 1;
  p.gamma = gamma;
  p.eps = eps;
  p.bcast = 0;
  p.out[0] = out;
  p.out_layout.ld = N;
  p.status = static_cast<fo::StatusWord*>(status32);
  p.timeout_ns = 20000000000ull;

  const char* why = nullptr;
  e = fo::launch_fused(g, p, s, &why);
  if (e != cudaSuccess) {
    char msg[200];
    std::snprintf(msg, sizeof(msg), "fo_gemm_rmsnorm_noalloc: launch failed: %s (%s)", cudaGetErrorString(e),
                  why ? why : "");
    return fail(7, err, err_len, msg);
  }
  return 0;
}
