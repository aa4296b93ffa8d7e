// RMSNorm and reorder+RMSNorm for 16-bit rows with fp32 statistics.
//
// One CTA of 256 threads per row; each thread owns 16-byte chunks
// (8 values) at stride 256 chunks.  Rows of up to 16384 values are held in
// registers between the statistics pass and the scaling pass; longer rows are
// read twice.  Unlike the reference kernels (reference: src/rmsnorm/rmsnorm.cuh:12-115,
// block size dim/16, eps fixed to 1e-5, default stream) any dim % 8 == 0 works,
// eps is an argument and the launch goes to the caller's stream.
#include "rmsnorm.h"

#include "gemm_fused_sm100.cuh"

namespace fo {

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormRegChunks = 8;

template <bool BF16, bool REORDER>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const uint16_t* __restrict__ x,
                                                               uint16_t* __restrict__ out,
                                                               const uint16_t* __restrict__ w, int rows, int dim,
                                                               float eps, OutLayout L) {
  __shared__ float red[kNormThreads / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int n_chunks = dim >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool in_regs = n_chunks <= kNormRegChunks * kNormThreads;

  auto src_ptr = [&](int c) -> const uint16_t* {
    if constexpr (REORDER) return x + layout_offset(L, row, c * 8);
    else return x + static_cast<long long>(row) * dim + c * 8;
  };

  uint4 v[kNormRegChunks];
  float ssq = 0.f;
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kNormRegChunks; ++k) {
      const int c = threadIdx.x + k * kNormThreads;
      if (c < n_chunks) v[k] = *reinterpret_cast<const uint4*>(src_ptr(c));
    }
#pragma unroll
    for (int k = 0; k < kNormRegChunks; ++k) {
      const int c = threadIdx.x + k * kNormThreads;
      if (c < n_chunks) {
        float2 f;
        f = unpack2<BF16>(v[k].x); ssq += f.x * f.x + f.y * f.y;
        f = unpack2<BF16>(v[k].y); ssq += f.x * f.x + f.y * f.y;
        f = unpack2<BF16>(v[k].z); ssq += f.x * f.x + f.y * f.y;
        f = unpack2<BF16>(v[k].w); ssq += f.x * f.x + f.y * f.y;
      }
    }
  } else {
    for (int c = threadIdx.x; c < n_chunks; c += kNormThreads) {
      const uint4 u = *reinterpret_cast<const uint4*>(src_ptr(c));
      float2 f;
      f = unpack2<BF16>(u.x); ssq += f.x * f.x + f.y * f.y;
      f = unpack2<BF16>(u.y); ssq += f.x * f.x + f.y * f.y;
      f = unpack2<BF16>(u.z); ssq += f.x * f.x + f.y * f.y;
      f = unpack2<BF16>(u.w); ssq += f.x * f.x + f.y * f.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
  if (lane == 0) red[warp] = ssq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / static_cast<float>(dim) + eps);

  auto emit = [&](int c, const uint4& u) {
    const uint4 g = *reinterpret_cast<const uint4*>(w + c * 8);
    float2 f;
    uint4 o;
    f = unpack2<BF16>(u.x); o.x = norm_pack2<BF16>(f.x, f.y, rstd, g.x);
    f = unpack2<BF16>(u.y); o.y = norm_pack2<BF16>(f.x, f.y, rstd, g.y);
    f = unpack2<BF16>(u.z); o.z = norm_pack2<BF16>(f.x, f.y, rstd, g.z);
    f = unpack2<BF16>(u.w); o.w = norm_pack2<BF16>(f.x, f.y, rstd, g.w);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(row) * dim + c * 8) = o;
  };
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kNormRegChunks; ++k) {
      const int c = threadIdx.x + k * kNormThreads;
      if (c < n_chunks) emit(c, v[k]);
    }
  } else {
    for (int c = threadIdx.x; c < n_chunks; c += kNormThreads) emit(c, *reinterpret_cast<const uint4*>(src_ptr(c)));
  }
}

template <bool REORDER>
cudaError_t launch(const void* x, void* out, const void* w, int rows, int dim, float eps, const OutLayout& L, DType dt,
                   cudaStream_t stream) {
  if (rows <= 0 || dim <= 0 || dim % 8 != 0) return cudaErrorInvalidValue;
  auto xs = reinterpret_cast<const uint16_t*>(x);
  auto os = reinterpret_cast<uint16_t*>(out);
  auto ws = reinterpret_cast<const uint16_t*>(w);
  if (dt == DT_BF16) rmsnorm_kernel<true, REORDER><<<rows, kNormThreads, 0, stream>>>(xs, os, ws, rows, dim, eps, L);
  else rmsnorm_kernel<false, REORDER><<<rows, kNormThreads, 0, stream>>>(xs, os, ws, rows, dim, eps, L);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_rmsnorm(const void* x, void* out, const void* w, int rows, int dim, float eps, DType dt,
                           cudaStream_t stream) {
  OutLayout L{};
  L.ld = dim;
  return launch<false>(x, out, w, rows, dim, eps, L, dt, stream);
}

cudaError_t launch_reorder_rmsnorm(const void* x, void* out, const void* w, int rows, int dim, float eps,
                                   const OutLayout& in_layout, DType dt, cudaStream_t stream) {
  if (in_layout.tiled && (in_layout.bn % 8 != 0 || in_layout.bm <= 0 || in_layout.rldn <= 0)) {
    return cudaErrorInvalidValue;
  }
  return launch<true>(x, out, w, rows, dim, eps, in_layout, dt, stream);
}

}  // namespace fo
