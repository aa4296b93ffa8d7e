// Launcher of the fused sm_100a GEMM kernel: builds the TMA descriptors,
// picks the template instance for (tile width, dtype) and launches one CTA per
// SM.  Counterpart of the reference's per-tile-config launchers
// (reference: src/gemm/gemm.cu:29-113, src/overlap/gemm_signal.cu:28-110,
// src/overlap/gemm_scatter.cu:28-111), without a workspace allocation.
#include "gemm_launch.h"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "gemm_fused_sm100.cuh"

namespace fo {

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

template <int BN, bool BF16, int CTAS>
cudaError_t launch_instance(const FusedParams& p, int grid, cudaStream_t stream) {
  using T = TileTraits<BN, CTAS>;
  auto kern = gemm_fused_sm100_kernel<BN, BF16, CTAS>;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  if (CTAS == 1) {
    kern<<<grid, kThreads, T::SMEM_BYTES, stream>>>(p);
    return cudaGetLastError();
  }
  // CTA pairs: a cluster of two CTAs per tile
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid & ~1), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

int device_sm_count() {
  static int cached[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && cached[dev] > 0) return cached[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 16) cached[dev] = n;
  return n;
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
  // every CTA stages 128 rows of A and (for a CTA pair) half of the B tile
  if (!make_tensor_map(&p.tmA, g.A, g.M, g.K, 128, g.dtype) ||
      !make_tensor_map(&p.tmB, g.B, g.N, g.K, tc.bn / tc.ctas, g.dtype)) {
    *why = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.TM = g.M / tc.bm;
  p.TN = g.N / tc.bn;
  if (p.raster_group <= 0) p.raster_group = 1;
  if (p.raster_group > p.TM) p.raster_group = p.TM;
  if (p.rot < 0 || p.rot >= p.TM) p.rot = 0;
  if (p.reduce && p.norm && static_cast<long long>(g.N) * 4 > TileTraits<256, 1>::STAGES * TileTraits<256, 1>::STAGE_BYTES + TileTraits<256, 1>::EPI_BYTES) {
    *why = "fused RMSNorm keeps a row in shared memory: N is too large (limit about 53000)";
    return cudaErrorInvalidValue;
  }
  int grid = g.sm_count > 0 ? g.sm_count : device_sm_count();
  const int sms = device_sm_count();
  if (grid > sms) grid = sms;  // every CTA must be resident: CTAs wait on one another's output
  if (p.reduce) {
    if (p.reduce_group != 1 && p.reduce_group != 2 && p.reduce_group != 4 && p.reduce_group != 8) {
      // Rows are latency-bound, so as many as possible should be in flight:
      // take the widest row group that still covers all owned rows in one
      // round (8 / G rows per CTA at a time).
      int gsel = 8;
      while (gsel > 1 && static_cast<long long>(grid) * (8 / gsel) < p.rows_per_owner) gsel >>= 1;
      p.reduce_group = gsel;
    }
    if (p.bcast) p.done_target *= static_cast<uint32_t>(p.reduce_group);  // one delivery count per warp and row
  }
  if (!p.reduce && !p.force_full_grid && grid > p.TM * p.TN * tc.ctas) grid = p.TM * p.TN * tc.ctas;
  if (tc.ctas == 2 && grid < 2) grid = 2;
  const bool bf16 = g.dtype == DT_BF16;
  if (tc.ctas == 2) {
    if (tc.bn == 256) {
      return bf16 ? launch_instance<256, true, 2>(p, grid, stream) : launch_instance<256, false, 2>(p, grid, stream);
    }
    return bf16 ? launch_instance<128, true, 2>(p, grid, stream) : launch_instance<128, false, 2>(p, grid, stream);
  }
  switch (tc.bn) {
    case 256:
      return bf16 ? launch_instance<256, true, 1>(p, grid, stream) : launch_instance<256, false, 1>(p, grid, stream);
    case 128:
      return bf16 ? launch_instance<128, true, 1>(p, grid, stream) : launch_instance<128, false, 1>(p, grid, stream);
    default:
      return bf16 ? launch_instance<64, true, 1>(p, grid, stream) : launch_instance<64, false, 1>(p, grid, stream);
  }
}

}  // namespace fo
