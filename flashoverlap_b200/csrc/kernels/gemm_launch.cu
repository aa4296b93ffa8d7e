// Launcher of the fused sm_100a GEMM kernel: builds the TMA descriptors,
// picks the template instance for (tile width, dtype) and launches one CTA per
// SM.  Counterpart of the reference's per-tile-config launchers
// (reference: src/gemm/gemm.cu:29-113, src/overlap/gemm_signal.cu:28-110,
// src/overlap/gemm_scatter.cu:28-111), without a workspace allocation.
#include "gemm_launch.h"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include <cstdlib>
#include <cstring>

#include "gemm_fused_sm100.cuh"

namespace fo {

#include "generated/algo_table.inc"

TileConfig algo_config(int algo) { return kAlgoTable[(algo < 0 || algo >= kNumAlgos) ? 0 : algo]; }

bool cooperative_launch_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("FLASHOVERLAP_COOPERATIVE");
    return e != nullptr && (std::strcmp(e, "1") == 0 || std::strcmp(e, "on") == 0);
  }();
  return on;
}

namespace {

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
  });
  return fn;
}

// 2-D row-major [rows, cols] 16-bit matrix, box = 64 columns x box_rows rows,
// 128-byte swizzle.  Out-of-range parts of a box read as zero.
bool make_tensor_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows, DType dt) {
  auto encode = get_encode_fn();
  if (encode == nullptr) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = encode(map, dt == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                      const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

int device_sm_count() {
  static int cached[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool slot = dev >= 0 && dev < kMaxDevices;
  if (slot && cached[dev] > 0) return cached[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (slot) cached[dev] = n;
  return n;
}

cudaError_t prepare_fused(int algo, DType dtype) {
  if (algo < 0 || algo >= kNumAlgos) return cudaErrorInvalidValue;
  return kPrepareTable[algo][dtype == DT_BF16 ? 1 : 0]();
}

cudaError_t launch_fused(const GemmOperands& g, FusedParams& p, cudaStream_t stream, const char** why) {
  const char* dummy;
  if (why == nullptr) why = &dummy;
  *why = "";
  const TileConfig tc = algo_config(g.algo);
  if (g.algo < 0 || g.algo >= kNumAlgos) {
    *why = "Algo index out of range";
    return cudaErrorInvalidValue;
  }
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.M % tc.bm != 0 || g.N % tc.bn != 0 || g.K % 8 != 0) {
    *why = "shape not supported: need M % tile_m == 0, N % tile_n == 0, K % 8 == 0";
    return cudaErrorInvalidValue;
  }
  if ((reinterpret_cast<uintptr_t>(g.A) & 15u) || (reinterpret_cast<uintptr_t>(g.B) & 15u)) {
    *why = "A and B must be 16-byte aligned";
    return cudaErrorInvalidValue;
  }
  // every CTA stages 128 rows of A and (for a CTA pair) half of the B tile, 64 K-values per box
  if (!make_tensor_map(&p.tmA, g.A, g.M, g.K, 128, g.dtype) ||
      !make_tensor_map(&p.tmB, g.B, g.N, g.K, tc.bn / tc.ctas, g.dtype)) {
    *why = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  p.a_own_begin = p.a_own_end = 0;
  if (g.A_own != nullptr && g.own_rows > 0) {
    if ((reinterpret_cast<uintptr_t>(g.A_own) & 15u) || g.own_begin < 0 || g.own_begin % 128 != 0 ||
        g.own_rows % 128 != 0 || g.own_begin + g.own_rows > g.M) {
      *why = "own rows of A must be 16-byte aligned whole blocks of 128 rows inside the matrix";
      return cudaErrorInvalidValue;
    }
    if (!make_tensor_map(&p.tmA_own, g.A_own, g.own_rows, g.K, 128, g.dtype)) {
      *why = "cuTensorMapEncodeTiled failed";
      return cudaErrorInvalidValue;
    }
    p.a_own_begin = g.own_begin;
    p.a_own_end = g.own_begin + g.own_rows;
  }
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.TM = g.M / tc.bm;
  p.TN = g.N / tc.bn;
  if (p.raster_group <= 0) p.raster_group = 1;
  if (p.raster_group > p.TM) p.raster_group = p.TM;
  if (p.rot < 0 || p.rot >= p.TM) p.rot = 0;
  int grid = g.sm_count > 0 ? g.sm_count : device_sm_count();
  const int sms = device_sm_count();
  if (grid > sms) grid = sms;  // every CTA must be resident: CTAs wait on one another's output
  if (p.reduce && p.job_counter == nullptr) {
    *why = "the reduce phase needs a row-job counter";
    return cudaErrorInvalidValue;
  }
  if (!p.reduce && !p.force_full_grid && grid > p.TM * p.TN * tc.ctas) grid = p.TM * p.TN * tc.ctas;
  if (tc.ctas == 2 && grid < 2) grid = 2;
  if (tc.ctas == 2) grid &= ~1;
  return kLaunchTable[g.algo][g.dtype == DT_BF16 ? 1 : 0](p, grid, stream);
}

}  // namespace fo
