// Registration of the library with PyTorch: two custom classes and the free
// operators, under the reference's namespaces (reference: src/pybind.cpp:114-150).
// Every method is registered under the upstream CUDA name and under the name
// used by the MUSA checkout of the reference, so that scripts written against
// either run unchanged.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <mutex>

#include <torch/custom_class.h>
#include <torch/library.h>

#include "../kernels/fused_params.h"
#include "../kernels/rmsnorm.h"
#include "baseline_impl.h"
#include "checks.h"
#include "overlap_impl.h"

namespace fo {

static std::vector<int64_t> generate_id_op() { return generate_nccl_id(); }

// reorder_rmsnorm(X, RX, RW, BM, BN, rldn, RA): X holds a [bs, dim] matrix in
// the tile-reordered layout, RX receives the RMS-normalised rows in natural
// order (reference: src/rmsnorm/rmsnorm.cpp:10-23, eps fixed to 1e-5 there).
static void reorder_rmsnorm_eps(at::Tensor X, at::Tensor RX, at::Tensor RW, int64_t BM, int64_t BN, int64_t rldn,
                                at::Tensor RA, double eps) {
  check_matrix(X, "X");
  check_matrix(RX, "RX");
  const DType dt = dtype_of(X);
  TORCH_CHECK(RX.scalar_type() == X.scalar_type() && RW.scalar_type() == X.scalar_type(), "dtype mismatch");
  TORCH_CHECK(RX.sizes() == X.sizes(), "RX must have the shape of X");
  const int64_t bs = X.size(0), dim = X.size(1);
  TORCH_CHECK(RW.is_cuda() && RW.is_contiguous() && RW.numel() == dim, "RW must hold dim values");
  TORCH_CHECK(BM > 0 && BN > 0 && bs % BM == 0 && dim % BN == 0 && BN % 8 == 0 && dim % 8 == 0,
              "need bs % BM == 0, dim % BN == 0, BN % 8 == 0");
  check_int_tensor(RA, "RA", true);
  const int64_t tiles = (bs / BM) * (dim / BN);
  TORCH_CHECK(RA.numel() == tiles, "RA must have ", tiles, " entries, got ", RA.numel());
  TORCH_CHECK(rldn >= 1 && tiles % rldn == 0, "rldn must divide the number of tiles");
  {  // the kernel gathers through RA: an entry outside [0, tiles) would read outside X
    static std::mutex mu;
    static IndexCheckCache checked;
    std::lock_guard<std::mutex> lock(mu);
    checked.require_permutation(RA, tiles, "RA");
  }
  OutLayout L{};
  L.tiled = 1;
  L.bm = static_cast<int>(BM);
  L.bn = static_cast<int>(BN);
  L.tn = static_cast<int>(dim / BN);
  L.rldn = static_cast<int>(rldn);
  L.ra = RA.data_ptr<int>();
  L.ld = dim;
  c10::cuda::CUDAGuard guard(X.device());
  cudaError_t e = launch_reorder_rmsnorm(X.data_ptr(), RX.data_ptr(), RW.data_ptr(), static_cast<int>(bs),
                                         static_cast<int>(dim), static_cast<float>(eps), L, dt,
                                         at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "reorder_rmsnorm launch failed: ", cudaGetErrorString(e));
}

static void reorder_rmsnorm_op(at::Tensor X, at::Tensor RX, at::Tensor RW, int64_t BM, int64_t BN, int64_t rldn,
                               at::Tensor RA) {
  reorder_rmsnorm_eps(X, RX, RW, BM, BN, rldn, RA, 1e-5);
}

// rmsnorm(X, O, RW, eps): exists in the reference's C++ (src/rmsnorm/rmsnorm.cpp:25-36)
// without being registered; registered here.
static void rmsnorm_op(at::Tensor X, at::Tensor O, at::Tensor RW, double eps) {
  check_matrix(X, "X");
  check_matrix(O, "O");
  const DType dt = dtype_of(X);
  TORCH_CHECK(O.scalar_type() == X.scalar_type() && RW.scalar_type() == X.scalar_type(), "dtype mismatch");
  TORCH_CHECK(O.sizes() == X.sizes(), "O must have the shape of X");
  TORCH_CHECK(RW.is_cuda() && RW.is_contiguous() && RW.numel() == X.size(1), "RW must hold dim values");
  TORCH_CHECK(X.size(1) % 8 == 0, "dim must be a multiple of 8");
  c10::cuda::CUDAGuard guard(X.device());
  cudaError_t e = launch_rmsnorm(X.data_ptr(), O.data_ptr(), RW.data_ptr(), static_cast<int>(X.size(0)),
                                 static_cast<int>(X.size(1)), static_cast<float>(eps), dt,
                                 at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "rmsnorm launch failed: ", cudaGetErrorString(e));
}

// The order in which the persistent kernel walks the tile grid, computed on
// the host by the function the kernel itself uses: entry i is
// tile_row * TN + tile_column of the i-th tile of the walk.  For tests and for
// tools that reason about completion order without a GPU.
static std::vector<int64_t> tile_walk_op(int64_t TM, int64_t TN, int64_t raster_group, bool taper, int64_t owner_stride,
                                         int64_t ws, int64_t me, int64_t rot) {
  TORCH_CHECK(TM > 0 && TN > 0 && TM * TN <= (1 << 24), "tile grid out of range");
  TORCH_CHECK(ws >= 1 && me >= 0 && me < ws && rot >= 0 && rot < TM, "rank or rotation out of range");
  TORCH_CHECK(owner_stride == 0 || owner_stride * ws == TM, "owner_stride must be TM / ws (or 0)");
  FusedParams p{};
  p.TM = static_cast<int>(TM);
  p.TN = static_cast<int>(TN);
  p.raster_group = static_cast<int>(raster_group < 1 ? 1 : (raster_group > TM ? TM : raster_group));
  p.raster_taper = taper ? 1 : 0;
  p.owner_stride = static_cast<int>(owner_stride);
  p.ws = static_cast<int>(ws);
  p.me = static_cast<int>(me);
  p.rot = static_cast<int>(rot);
  std::vector<int64_t> out(static_cast<size_t>(TM * TN));
  for (int t = 0; t < p.TM * p.TN; ++t) {
    int m_blk = 0, n_blk = 0;
    tile_coords(p, t, m_blk, n_blk);
    out[static_cast<size_t>(t)] = static_cast<int64_t>(m_blk) * TN + n_blk;
  }
  return out;
}

}  // namespace fo

TORCH_LIBRARY(flashoverlap_class, m) {
  using fo::BaselineImpl;
  using fo::OverlapImpl;
  m.class_<BaselineImpl>("BaselineImpl")
      .def(torch::init<>())
      .def("nccl_init", &BaselineImpl::NcclInit)
      .def("mccl_init", &BaselineImpl::NcclInit)
      .def("cublas_init", &BaselineImpl::CublasInit)
      .def("mublas_init", &BaselineImpl::CublasInit)
      .def("gemm_allreduce", &BaselineImpl::GemmAllReduce)
      .def("gemm_reducescatter", &BaselineImpl::GemmReduceScatter)
      .def("gemm_all2all", &BaselineImpl::GemmAll2All)
      .def("cublas_gemm", &BaselineImpl::Gemm)
      .def("mublas_gemm", &BaselineImpl::Gemm)
      .def("nccl_allreduce", &BaselineImpl::NcclAllReduce)
      .def("mccl_allreduce", &BaselineImpl::NcclAllReduce)
      .def("nccl_reducescatter", &BaselineImpl::NcclReduceScatter)
      .def("mccl_reducescatter", &BaselineImpl::NcclReduceScatter)
      .def("nccl_all2all", &BaselineImpl::NcclAll2All)
      .def("mccl_all2all", &BaselineImpl::NcclAll2All);

  m.class_<OverlapImpl>("OverlapImpl")
      .def(torch::init<>())
      .def("nccl_init", &OverlapImpl::NcclInit)
      .def("mccl_init", &OverlapImpl::NcclInit)
      .def("cutlass_init", &OverlapImpl::CutlassInit)
      .def("mutlass_init", &OverlapImpl::CutlassInit)
      .def("overlap_init", &OverlapImpl::OverlapInit)
      .def("cutlass_gemm", &OverlapImpl::Gemm)
      .def("mutlass_gemm", &OverlapImpl::Gemm)
      .def("gemm_allreduce_overlap", &OverlapImpl::GemmAllReduceOverlap)
      .def("gemm_reducescatter_overlap", &OverlapImpl::GemmReduceScatterOverlap)
      .def("gemm_allreduce", &OverlapImpl::GemmAllReduce)
      .def("gemm_reducescatter", &OverlapImpl::GemmReduceScatter)
      .def("gemm_all2all", &OverlapImpl::GemmAll2All)
      .def("nccl_allreduce", &OverlapImpl::NcclAllReduce)
      .def("mccl_allreduce", &OverlapImpl::NcclAllReduce)
      .def("nccl_reducescatter", &OverlapImpl::NcclReduceScatter)
      .def("mccl_reducescatter", &OverlapImpl::NcclReduceScatter)
      .def("nccl_all2all", &OverlapImpl::NcclAll2All)
      .def("mccl_all2all", &OverlapImpl::NcclAll2All)
      .def("seg_allreduce", &OverlapImpl::SegAllReduce)
      .def("gemm_allreduce_twostream", &OverlapImpl::GemmAllReduceTwoStream)
      .def("gemm_reducescatter_twostream", &OverlapImpl::GemmReduceScatterTwoStream)
      .def("gemm_allreduce_fused", &OverlapImpl::GemmAllReduceFused)
      .def("gemm_reducescatter_fused", &OverlapImpl::GemmReduceScatterFused)
      .def("gemm_rmsnorm", &OverlapImpl::GemmRmsNorm)
      .def("allgather_gemm", &OverlapImpl::AllGatherGemm)
      .def("a2a_dispatch_gemm", &OverlapImpl::A2aDispatchGemm)
      .def("a2a_padded_rows", &OverlapImpl::A2aPaddedRows)
      .def("attach_symmetric", &OverlapImpl::AttachSymmetric)
      .def("detach_symmetric", &OverlapImpl::DetachSymmetric)
      .def("set_use_nvls", &OverlapImpl::SetUseNvls)
      .def("set_allgather_multicast", &OverlapImpl::SetAllGatherMulticast)
      .def("nvls_available", &OverlapImpl::NvlsAvailable)
      .def("allreduce_uses_nvls", &OverlapImpl::AllReduceUsesNvls)
      .def("p2p_push", &OverlapImpl::P2pPush)
      .def("p2p_push_bulk", &OverlapImpl::P2pPushBulk)
      .def("multimem_bench", &OverlapImpl::MultimemBench)
      .def("wait_on_unset_counter", &OverlapImpl::WaitOnUnsetCounter)
      .def("set_transport", &OverlapImpl::SetTransport)
      .def("transport", &OverlapImpl::Transport)
      .def("set_timeout_ms", &OverlapImpl::SetTimeoutMs)
      .def("set_sm_count", &OverlapImpl::SetSmCount)
      .def("set_raster_group", &OverlapImpl::SetRasterGroup)
      .def("set_l2_hints", &OverlapImpl::SetL2Hints)
      .def("set_raster_taper", &OverlapImpl::SetRasterTaper)
      .def("set_phase_trace", &OverlapImpl::SetPhaseTrace)
      .def("set_row_trace", &OverlapImpl::SetRowTrace)
      .def("status", &OverlapImpl::Status)
      .def("status_string", &OverlapImpl::StatusString)
      .def("check_status", &OverlapImpl::CheckStatus)
      .def("reset", &OverlapImpl::Reset)
      .def("num_algos", &OverlapImpl::NumAlgos)
      .def("algo_tile", &OverlapImpl::AlgoTile);
}

TORCH_LIBRARY(flashoverlap_op, m) {
  m.def("generate_nccl_id", &fo::generate_id_op);
  m.def("generate_mccl_id", &fo::generate_id_op);
  m.def("reorder_rmsnorm", &fo::reorder_rmsnorm_op);
  m.def("reorder_rmsnorm_eps", &fo::reorder_rmsnorm_eps);
  m.def("rmsnorm", &fo::rmsnorm_op);
  m.def("tile_walk", &fo::tile_walk_op);
}
