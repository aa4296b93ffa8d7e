#include "overlap_impl.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cuda.h>
#include <nvtx3/nvToolsExt.h>
#include <unistd.h>

#include <functional>

#include "../kernels/comm_kernels.h"
#include "../kernels/rmsnorm.h"
#include "checks.h"

namespace fo {

namespace {

ncclDataType_t nccl_type(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16 ? ncclBfloat16 : ncclHalf; }

cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// Validates the reference's reorder/segment arguments and returns the layout
// they describe for an M x N matrix (tile shape from RA's 2-D shape).
OutLayout tiled_layout(int64_t M, int64_t N, const at::Tensor& RA, int64_t rLDN, int64_t algo,
                       IndexCheckCache& checked) {
  check_int_tensor(RA, "RA", true);
  TORCH_CHECK(RA.dim() == 2, "RA must be 2-D [M/BM, N/BN]");
  const int64_t tm = RA.size(0), tn = RA.size(1);
  TORCH_CHECK(tm > 0 && tn > 0 && M % tm == 0 && N % tn == 0, "RA shape ", tm, "x", tn, " does not divide M x N");
  const TileConfig tc = algo_config(static_cast<int>(algo));
  TORCH_CHECK(M / tm == tc.bm && N / tn == tc.bn, "RA describes ", M / tm, "x", N / tn, " tiles but Algo ", algo,
              " computes ", tc.bm, "x", tc.bn, " tiles");
  TORCH_CHECK(rLDN >= 1 && (tm * tn) % rLDN == 0, "rLDN must divide the number of tiles");
  checked.require_permutation(RA, tm * tn, "RA");  // the kernels store through RA
  OutLayout L{};
  L.tiled = 1;
  L.bm = tc.bm;
  L.bn = tc.bn;
  L.tn = static_cast<int>(tn);
  L.rldn = static_cast<int>(rLDN);
  L.ra = RA.data_ptr<int>();
  L.ld = N;
  return L;
}

void check_segments(const at::Tensor& cSEG_CPU, const at::Tensor& cSEG_GPU, int64_t tiles, const at::Tensor& MM,
                    int64_t tn, bool monitor) {
  check_int_tensor(cSEG_CPU, "cSEG_CPU", false);
  check_int_tensor(cSEG_GPU, "cSEG_GPU", true);
  check_int_tensor(MM, "MM", true);
  TORCH_CHECK(cSEG_CPU.numel() == cSEG_GPU.numel(), "cSEG_CPU and cSEG_GPU differ in length");
  TORCH_CHECK(cSEG_CPU.numel() >= 1, "cSeg is empty");
  int64_t sum = 0;
  const int* seg = cSEG_CPU.data_ptr<int>();
  for (int64_t i = 0; i < cSEG_CPU.numel(); ++i) {
    TORCH_CHECK(seg[i] > 0, "cSeg[", i, "] must be positive");
    sum += seg[i];
  }
  TORCH_CHECK(sum == tiles, "sum(cSeg) = ", sum, " but the GEMM has ", tiles, " tiles");
  TORCH_CHECK(MM.numel() >= cSEG_CPU.numel(), "MM has ", MM.numel(), " counters, fewer than the ", cSEG_CPU.numel(),
              " segments");
  if (monitor) {
    TORCH_CHECK(MM.numel() >= tn + tiles, "monitor mode needs MM of shape (M/BM + 1, N/BN): ", tn + tiles,
                " entries, got ", MM.numel());
    TORCH_CHECK(cSEG_CPU.numel() < tn, "monitor mode keeps its ticket in MM[N/BN - 1]; use fewer than ", tn,
                " segments");
  }
}

}  // namespace

OverlapImpl::OverlapImpl() = default;
OverlapImpl::~OverlapImpl() {
  if (join_event_ != nullptr) cudaEventDestroy(join_event_);
  if (raise_event_ != nullptr) cudaEventDestroy(raise_event_);
  if (comm_stream_ != nullptr) cudaStreamDestroy(comm_stream_);
}

void OverlapImpl::require_comm(const char* op) const {
  TORCH_CHECK(comm_.world() == 1 || comm_.active(), op, ": call nccl_init first");
}

GemmOperands OverlapImpl::operands(const at::Tensor& A, const at::Tensor& B, int64_t algo) const {
  TORCH_CHECK(algo >= 0 && algo < kNumAlgos, "Algo must be in [0, ", kNumAlgos, "), got ", algo);
  GemmOperands g{};
  g.A = A.data_ptr();
  g.B = B.data_ptr();
  g.M = static_cast<int>(A.size(0));
  g.N = static_cast<int>(B.size(0));
  g.K = static_cast<int>(A.size(1));
  g.dtype = dtype_of(A);
  g.algo = static_cast<int>(algo);
  g.sm_count = 0;
  const TileConfig tc = algo_config(g.algo);
  TORCH_CHECK(g.M % tc.bm == 0 && g.N % tc.bn == 0, "M must be a multiple of ", tc.bm, " and N of ", tc.bn,
              " for Algo ", algo, " (got M=", g.M, ", N=", g.N, ")");
  TORCH_CHECK(g.K % 8 == 0, "K must be a multiple of 8, got ", g.K);
  return g;
}

void OverlapImpl::NcclInit(int64_t rank, int64_t size, std::vector<int64_t> id) {
  comm_.init(static_cast<int>(rank), static_cast<int>(size), id);
  // Ranks on different hosts cannot map each other's memory: keep them on NCCL.
  if (size > 1) {
    char host[256] = {};
    gethostname(host, sizeof(host) - 1);
    const uint64_t mine = std::hash<std::string>{}(std::string(host));
    std::vector<uint64_t> all(static_cast<size_t>(size));
    comm_.all_gather_host(&mine, sizeof(mine), all.data());
    for (uint64_t h : all) nccl_transport_ = nccl_transport_ || h != mine;
  }
  const Communicator* c = &comm_;
  engine_.init(static_cast<int>(rank), static_cast<int>(size),
               [c](const void* send, size_t bytes, void* recv) { c->all_gather_host(send, bytes, recv); });
  engine_ready_ = true;
}

void OverlapImpl::CutlassInit() {
  // The reference captures the current stream here (reference:
  // src/overlap_impl.cu:38-40).  Every operation below uses the stream that is
  // current when it is called, so there is nothing to capture.
  if (!engine_ready_) {
    engine_.init(0, 1, nullptr);
    engine_ready_ = true;
  }
}

void OverlapImpl::OverlapInit() {
  // The reference creates its communication stream here (reference:
  // src/overlap_impl.cu:146-148); the fused kernel needs no second stream.
  if (!engine_ready_) {
    engine_.init(0, 1, nullptr);
    engine_ready_ = true;
  }
}

void OverlapImpl::Gemm(at::Tensor A, at::Tensor B, at::Tensor C, int64_t algo) {
  check_gemm_args(A, B, &C);
  c10::cuda::CUDAGuard guard(A.device());
  engine_.gemm(operands(A, B, algo), C.data_ptr(), nullptr, nullptr, current_stream());
}

void OverlapImpl::GemmAllReduceOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor MM, at::Tensor RA,
                                       int64_t rLDN, at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t algo,
                                       bool if_monitor) {
  check_gemm_args(A, B, &C);
  require_comm("gemm_allreduce_overlap");
  c10::cuda::CUDAGuard guard(A.device());
  GemmOperands g = operands(A, B, algo);
  OutLayout L = tiled_layout(g.M, g.N, RA, rLDN, algo, index_checks_);
  const int64_t tiles = RA.numel();
  check_segments(cSEG_CPU, cSEG_GPU, tiles, MM, RA.size(1), if_monitor);
  if (nccl_transport_) {
    two_stream(false, A, B, C, nullptr, MM, RA, nullptr, rLDN, cSEG_CPU, cSEG_GPU, algo, 0, if_monitor);
    return;
  }
  cudaStream_t stream = current_stream();
  SignalArgs sig;
  if (if_monitor) {
    // Completion-order trace of the GEMM tiles, in the reference's format:
    // MM[N/BN - 1] is the ticket counter, MM[N/BN + slot] the ticket of the
    // tile stored in `slot` (reference: src/overlap/gemm_with_signal.h:197-200).
    sig.ticket_counter = MM.data_ptr<int>() + (RA.size(1) - 1);
    sig.trace = MM.data_ptr<int>() + RA.size(1);
    sig.slot_of_tile = RA.data_ptr<int>();
  }
  engine_.gemm_allreduce(g, C.data_ptr(), NormArgs{}, &L, if_monitor ? &sig : nullptr, stream);
}

void OverlapImpl::GemmReduceScatterOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor MM,
                                           at::Tensor RA, at::Tensor RE, int64_t rLDN, at::Tensor cSEG_CPU,
                                           at::Tensor cSEG_GPU, int64_t algo, bool if_monitor) {
  check_gemm_args(A, B, &C);
  require_comm("gemm_reducescatter_overlap");
  c10::cuda::CUDAGuard guard(A.device());
  GemmOperands g = operands(A, B, algo);
  const int ws = comm_.world();
  OutLayout L = tiled_layout(g.M, g.N, RA, rLDN, algo, index_checks_);
  const int64_t tiles = RA.numel();
  check_segments(cSEG_CPU, cSEG_GPU, tiles, MM, RA.size(1), if_monitor);
  check_int_tensor(RE, "RE", true);
  TORCH_CHECK(RE.numel() == static_cast<int64_t>(g.M) * g.N / L.bn, "RE must have M*N/BN = ",
              static_cast<int64_t>(g.M) * g.N / L.bn, " entries, got ", RE.numel());
  index_checks_.require_range(RE, RE.numel(), "RE");
  TORCH_CHECK(L.bm % ws == 0, "BM must be divisible by the world size");
  check_matrix(D, "D");
  TORCH_CHECK(D.scalar_type() == A.scalar_type() && D.numel() == static_cast<int64_t>(g.M) * g.N / ws,
              "D must hold M*N/size elements of A's dtype");
  if (nccl_transport_) {
    two_stream(true, A, B, C, &D, MM, RA, &RE, rLDN, cSEG_CPU, cSEG_GPU, algo, 0, if_monitor);
    return;
  }
  cudaStream_t stream = current_stream();
  SignalArgs sig;
  if (if_monitor) {
    sig.ticket_counter = MM.data_ptr<int>() + (RA.size(1) - 1);
    sig.trace = MM.data_ptr<int>() + RA.size(1);
    sig.slot_of_tile = RA.data_ptr<int>();
  }
  // Rank r keeps the rows m with m % size == r of every tile; D is the
  // (M/size) x N matrix of those rows in the same slot order with tiles of
  // BM/size rows (reference: src/overlap/gemm_with_scatter.h:161-177 together
  // with the per-segment reduce-scatter, src/overlap_impl.cu:314-321).
  OutLayout LD = L;
  LD.bm = L.bm / ws;
  engine_.gemm_reducescatter(g, D.data_ptr(), /*interleave=*/true, NormArgs{}, &LD, if_monitor ? &sig : nullptr, stream);
}

void OverlapImpl::GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C, int64_t algo) {
  check_gemm_args(A, B, &C);
  require_comm("gemm_allreduce");
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = current_stream();
  engine_.gemm(operands(A, B, algo), C.data_ptr(), nullptr, nullptr, stream);
  if (comm_.active()) {
    FO_NCCL_CHECK(ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
  }
}

void OverlapImpl::GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t algo) {
  check_gemm_args(A, B, &C);
  require_comm("gemm_reducescatter");
  c10::cuda::CUDAGuard guard(A.device());
  const int ws = comm_.world();
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && D.scalar_type() == C.scalar_type() && D.numel() * ws == C.numel(),
              "D must hold M*N/size elements of C's dtype");
  cudaStream_t stream = current_stream();
  engine_.gemm(operands(A, B, algo), C.data_ptr(), nullptr, nullptr, stream);
  if (comm_.active()) {
    FO_NCCL_CHECK(ncclReduceScatter(C.data_ptr(), D.data_ptr(), D.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
  } else {
    FO_CUDA_CHECK(cudaMemcpyAsync(D.data_ptr(), C.data_ptr(), C.nbytes(), cudaMemcpyDeviceToDevice, stream));
  }
}

namespace {
// Pairwise exchange of row blocks: rank i sends mLen[i][j] rows (of `width`
// values) to rank j; chunks are packed in peer order, skipping self, on both
// sides (reference: src/overlap_impl.cu:128-141).
void all2all_rows(const Communicator& comm, const at::Tensor& C, at::Tensor& D, const at::Tensor& mLen,
                  int64_t width, cudaStream_t stream) {
  const int ws = comm.world(), rank = comm.rank();
  check_int_tensor(mLen, "mLen_CPU", false);
  TORCH_CHECK(mLen.numel() == static_cast<int64_t>(ws) * ws, "mLen_CPU must be [size, size]");
  const int* len = mLen.data_ptr<int>();
  int64_t send_rows = 0, recv_rows = 0;
  for (int peer = 0; peer < ws; ++peer) {
    if (peer == rank) continue;
    TORCH_CHECK(len[rank * ws + peer] >= 0 && len[peer * ws + rank] >= 0, "mLen_CPU entries must be >= 0");
    send_rows += len[rank * ws + peer];
    recv_rows += len[peer * ws + rank];
  }
  TORCH_CHECK(send_rows * width <= C.numel(), "send chunks (", send_rows, " rows) exceed C");
  TORCH_CHECK(recv_rows * width <= D.numel(), "receive chunks (", recv_rows, " rows) exceed D");
  if (!comm.active()) return;
  const size_t esz = C.element_size();
  char* src = static_cast<char*>(C.data_ptr());
  char* dst = static_cast<char*>(D.data_ptr());
  FO_NCCL_CHECK(ncclGroupStart());
  for (int peer = 0; peer < ws; ++peer) {
    if (peer == rank) continue;
    const size_t n_send = static_cast<size_t>(len[rank * ws + peer]) * width;
    const size_t n_recv = static_cast<size_t>(len[peer * ws + rank]) * width;
    FO_NCCL_CHECK(ncclSend(src, n_send, nccl_type(C), peer, comm.get(), stream));
    FO_NCCL_CHECK(ncclRecv(dst, n_recv, nccl_type(C), peer, comm.get(), stream));
    src += n_send * esz;
    dst += n_recv * esz;
  }
  FO_NCCL_CHECK(ncclGroupEnd());
}
}  // namespace

void OverlapImpl::GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t algo,
                              at::Tensor mLen_CPU) {
  check_gemm_args(A, B, &C);
  require_comm("gemm_all2all");
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && D.scalar_type() == C.scalar_type(), "D must match C's dtype");
  cudaStream_t stream = current_stream();
  engine_.gemm(operands(A, B, algo), C.data_ptr(), nullptr, nullptr, stream);
  all2all_rows(comm_, C, D, mLen_CPU, B.size(0), stream);
}

void OverlapImpl::NcclAllReduce(at::Tensor C) {
  require_comm("nccl_allreduce");
  TORCH_CHECK(C.is_cuda() && C.is_contiguous(), "C must be a contiguous CUDA tensor");
  dtype_of(C);
  c10::cuda::CUDAGuard guard(C.device());
  if (!comm_.active()) return;
  FO_NCCL_CHECK(
      ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_type(C), ncclSum, comm_.get(), current_stream()));
}

void OverlapImpl::NcclReduceScatter(at::Tensor C) {
  require_comm("nccl_reducescatter");
  TORCH_CHECK(C.is_cuda() && C.is_contiguous(), "C must be a contiguous CUDA tensor");
  dtype_of(C);
  c10::cuda::CUDAGuard guard(C.device());
  if (!comm_.active()) return;
  const int ws = comm_.world();
  TORCH_CHECK(C.numel() % ws == 0, "C.numel() must be divisible by the world size");
  const size_t count = C.numel() / ws;
  char* recv = static_cast<char*>(C.data_ptr()) + static_cast<size_t>(comm_.rank()) * count * C.element_size();
  FO_NCCL_CHECK(ncclReduceScatter(C.data_ptr(), recv, count, nccl_type(C), ncclSum, comm_.get(), current_stream()));
}

void OverlapImpl::NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU) {
  require_comm("nccl_all2all");
  TORCH_CHECK(C.is_cuda() && C.is_contiguous() && C.dim() == 2, "C must be a contiguous 2-D CUDA tensor");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && D.scalar_type() == C.scalar_type(), "D must match C's dtype");
  dtype_of(C);
  c10::cuda::CUDAGuard guard(C.device());
  all2all_rows(comm_, C, D, mLen_CPU, C.size(1), current_stream());
}

void OverlapImpl::SegAllReduce(at::Tensor C, at::Tensor cSEG_CPU, int64_t SegNum) {
  require_comm("seg_allreduce");
  TORCH_CHECK(C.is_cuda() && C.is_contiguous(), "C must be a contiguous CUDA tensor");
  dtype_of(C);
  check_int_tensor(cSEG_CPU, "cSEG_CPU", false);
  TORCH_CHECK(SegNum > 0 && C.numel() % SegNum == 0, "SegNum must divide C.numel()");
  const int* seg = cSEG_CPU.data_ptr<int>();
  int64_t sum = 0;
  for (int64_t i = 0; i < cSEG_CPU.numel(); ++i) sum += seg[i];
  TORCH_CHECK(sum <= SegNum, "sum(cSeg) = ", sum, " exceeds SegNum = ", SegNum);
  c10::cuda::CUDAGuard guard(C.device());
  if (!comm_.active()) return;
  const size_t unit = C.numel() / SegNum;
  char* base = static_cast<char*>(C.data_ptr());
  size_t done = 0;
  for (int64_t i = 0; i < cSEG_CPU.numel(); ++i) {
    const size_t n = unit * static_cast<size_t>(seg[i]);
    char* ptr = base + done * C.element_size();
    FO_NCCL_CHECK(ncclAllReduce(ptr, ptr, n, nccl_type(C), ncclSum, comm_.get(), current_stream()));
    done += n;
  }
}

namespace {
using StreamWaitFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
StreamWaitFn stream_wait_value32() {
  static StreamWaitFn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    looked = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<StreamWaitFn>(ptr);
    }
  }
  return fn;
}
}  // namespace

void OverlapImpl::two_stream(bool scatter, at::Tensor& A, at::Tensor& B, at::Tensor& C, at::Tensor* D, at::Tensor& MM,
                             at::Tensor& RA, at::Tensor* RE, int64_t rLDN, at::Tensor& cSEG_CPU, at::Tensor& cSEG_GPU,
                             int64_t algo, int64_t gemm_ctas, bool monitor) {
  nvtxRangePushA(scatter ? "flashoverlap::two_stream_reducescatter" : "flashoverlap::two_stream_allreduce");
  struct Pop {
    ~Pop() { nvtxRangePop(); }
  } pop;
  check_gemm_args(A, B, &C);
  require_comm("two-stream overlap");
  c10::cuda::CUDAGuard guard(A.device());
  GemmOperands g = operands(A, B, algo);
  OutLayout L = tiled_layout(g.M, g.N, RA, rLDN, algo, index_checks_);
  const int64_t tiles = RA.numel();
  check_segments(cSEG_CPU, cSEG_GPU, tiles, MM, RA.size(1), monitor);
  const int ws = comm_.world();
  const TileConfig tc = algo_config(g.algo);
  if (scatter) {
    TORCH_CHECK(D != nullptr && RE != nullptr, "reduce-scatter needs D and RE");
    check_int_tensor(*RE, "RE", true);
    TORCH_CHECK(D->is_cuda() && D->is_contiguous() && D->scalar_type() == A.scalar_type() &&
                    D->numel() * ws == C.numel(),
                "D must hold M*N/size elements of A's dtype");
    TORCH_CHECK(L.bm % ws == 0, "BM must be divisible by the world size");
    TORCH_CHECK(rLDN == 1, "the row map is defined for rLDN == 1");
    TORCH_CHECK(RE->numel() == static_cast<int64_t>(g.M) * g.N / L.bn, "RE must have M*N/BN entries");
    index_checks_.require_range(*RE, RE->numel(), "RE");  // the epilogue stores through this map
  }
  auto wait_fn = stream_wait_value32();
  TORCH_CHECK(wait_fn != nullptr, "cuStreamWaitValue32 is not available from this driver");
  if (comm_stream_ == nullptr) {
    int lo = 0, hi = 0;
    FO_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    FO_CUDA_CHECK(cudaStreamCreateWithPriority(&comm_stream_, cudaStreamNonBlocking, hi));
    FO_CUDA_CHECK(cudaEventCreateWithFlags(&join_event_, cudaEventDisableTiming));
    FO_CUDA_CHECK(cudaEventCreateWithFlags(&raise_event_, cudaEventDisableTiming));
  }
  cudaStream_t stream = current_stream();
  // the collectives may start only after earlier work on the caller's stream (inputs, previous use of C / MM)
  FO_CUDA_CHECK(cudaEventRecord(join_event_, stream));
  FO_CUDA_CHECK(cudaStreamWaitEvent(comm_stream_, join_event_, 0));

  SignalArgs sig;
  sig.seg_counter = MM.data_ptr<int>();
  sig.cseg = cSEG_GPU.data_ptr<int>();
  sig.nseg = static_cast<int>(cSEG_GPU.numel());
  sig.slot_of_tile = RA.data_ptr<int>();
  if (monitor) {  // completion tickets in the reference's MM layout
    sig.ticket_counter = MM.data_ptr<int>() + (RA.size(1) - 1);
    sig.trace = MM.data_ptr<int>() + RA.size(1);
  }
  int ctas = static_cast<int>(gemm_ctas);
  if (ctas <= 0) ctas = device_sm_count() - 16;
  if (tc.ctas == 2) ctas &= ~1;
  TORCH_CHECK(ctas >= tc.ctas, "too few CTAs for the GEMM");
  g.sm_count = ctas;
  // the segment counters start from zero whatever an earlier (possibly aborted) call left in them
  FO_CUDA_CHECK(cudaMemsetAsync(MM.data_ptr<int>(), 0, sizeof(int) * cSEG_CPU.numel(), stream));
  if (scatter) {
    // rows of every tile grouped by (row % size), segment by segment: what the
    // reference's scatter epilogue writes through its row map RE
    OutLayout LS = L;
    LS.row_map = RE->data_ptr<int>();
    engine_.gemm(g, C.data_ptr(), &LS, &sig, stream);
  } else {
    engine_.gemm(g, C.data_ptr(), &L, &sig, stream);
  }
  // The stream waits below have no deadline of their own.  This kernel runs on
  // the caller's stream right after the GEMM and raises every segment counter
  // to its target, so the waits end when the GEMM has ended, also when the
  // GEMM gave up on one of its bounded waits (its status word then says so).
  FO_CUDA_CHECK(launch_raise_counters(MM.data_ptr<int>(), cSEG_GPU.data_ptr<int>(), tc.ctas,
                                      static_cast<int>(cSEG_CPU.numel()), stream));
  FO_CUDA_CHECK(cudaEventRecord(raise_event_, stream));
  const int* seg = cSEG_CPU.data_ptr<int>();
  const size_t tile_elems = static_cast<size_t>(L.bm) * L.bn;
  const size_t esz = C.element_size();
  size_t done = 0;
  for (int64_t i = 0; i < cSEG_CPU.numel(); ++i) {
    const size_t count = tile_elems * static_cast<size_t>(seg[i]);
    CUresult r = wait_fn(reinterpret_cast<CUstream>(comm_stream_),
                         reinterpret_cast<CUdeviceptr>(MM.data_ptr<int>() + i),
                         static_cast<cuuint32_t>(seg[i] * tc.ctas), CU_STREAM_WAIT_VALUE_GEQ);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuStreamWaitValue32 failed with ", static_cast<int>(r));
    char* src = static_cast<char*>(C.data_ptr()) + done * esz;
    if (comm_.active()) {
      if (scatter) {
        char* dst = static_cast<char*>(D->data_ptr()) + done / ws * esz;
        FO_NCCL_CHECK(ncclReduceScatter(src, dst, count / ws, nccl_type(C), ncclSum, comm_.get(), comm_stream_));
      } else {
        FO_NCCL_CHECK(ncclAllReduce(src, src, count, nccl_type(C), ncclSum, comm_.get(), comm_stream_));
      }
    } else if (scatter) {
      FO_CUDA_CHECK(cudaMemcpyAsync(D->data_ptr(), C.data_ptr(), C.nbytes(), cudaMemcpyDeviceToDevice, comm_stream_));
    }
    done += count;
  }
  // the counters return to zero (the reference's wait kernel swaps them back on success), after the raise
  FO_CUDA_CHECK(cudaStreamWaitEvent(comm_stream_, raise_event_, 0));
  FO_CUDA_CHECK(cudaMemsetAsync(MM.data_ptr<int>(), 0, sizeof(int) * cSEG_CPU.numel(), comm_stream_));
  FO_CUDA_CHECK(cudaEventRecord(join_event_, comm_stream_));
  FO_CUDA_CHECK(cudaStreamWaitEvent(stream, join_event_, 0));
}

void OverlapImpl::GemmAllReduceTwoStream(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor MM, at::Tensor RA,
                                         int64_t rLDN, at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t algo,
                                         int64_t gemm_ctas) {
  two_stream(false, A, B, C, nullptr, MM, RA, nullptr, rLDN, cSEG_CPU, cSEG_GPU, algo, gemm_ctas, false);
}

void OverlapImpl::GemmReduceScatterTwoStream(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor MM,
                                             at::Tensor RA, at::Tensor RE, int64_t rLDN, at::Tensor cSEG_CPU,
                                             at::Tensor cSEG_GPU, int64_t algo, int64_t gemm_ctas) {
  two_stream(true, A, B, C, &D, MM, RA, &RE, rLDN, cSEG_CPU, cSEG_GPU, algo, gemm_ctas, false);
}

at::Tensor OverlapImpl::GemmAllReduceFused(at::Tensor A, at::Tensor B, c10::optional<at::Tensor> weight, double eps,
                                           int64_t algo) {
  check_gemm_args(A, B, nullptr);
  require_comm("gemm_allreduce_fused");
  TORCH_CHECK(engine_ready_, "gemm_allreduce_fused: call nccl_init first");
  c10::cuda::CUDAGuard guard(A.device());
  GemmOperands g = operands(A, B, algo);
  NormArgs norm;
  if (weight.has_value()) {
    TORCH_CHECK(weight->is_cuda() && weight->is_contiguous() && weight->numel() == g.N &&
                    weight->scalar_type() == A.scalar_type(),
                "weight must be a contiguous CUDA tensor of N values with A's dtype");
    norm.gamma = weight->data_ptr();
    norm.eps = static_cast<float>(eps);
  }
  if (nccl_transport_) {
    cudaStream_t stream = current_stream();
    at::Tensor C = torch::empty({g.M, g.N}, A.options());
    engine_.gemm(g, C.data_ptr(), nullptr, nullptr, stream);
    FO_NCCL_CHECK(ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
    if (norm.gamma != nullptr) {
      at::Tensor O = torch::empty_like(C);
      FO_CUDA_CHECK(launch_rmsnorm(C.data_ptr(), O.data_ptr(), norm.gamma, g.M, g.N, norm.eps, g.dtype, stream));
      return O;
    }
    return C;
  }
  void* res = engine_.gemm_allreduce(g, nullptr, norm, nullptr, nullptr, current_stream());
  return torch::from_blob(res, {g.M, g.N}, A.options());
}

void OverlapImpl::GemmReduceScatterFused(at::Tensor A, at::Tensor B, at::Tensor D, c10::optional<at::Tensor> weight,
                                         double eps, int64_t algo, bool interleave) {
  check_gemm_args(A, B, nullptr);
  require_comm("gemm_reducescatter_fused");
  TORCH_CHECK(engine_ready_, "gemm_reducescatter_fused: call nccl_init first");
  c10::cuda::CUDAGuard guard(A.device());
  GemmOperands g = operands(A, B, algo);
  const int ws = comm_.world();
  check_matrix(D, "D");
  TORCH_CHECK(D.scalar_type() == A.scalar_type() && D.size(0) * ws == g.M && D.size(1) == g.N,
              "D must be [M/size, N] with A's dtype");
  NormArgs norm;
  if (weight.has_value()) {
    TORCH_CHECK(weight->is_cuda() && weight->is_contiguous() && weight->numel() == g.N &&
                    weight->scalar_type() == A.scalar_type(),
                "weight must be a contiguous CUDA tensor of N values with A's dtype");
    norm.gamma = weight->data_ptr();
    norm.eps = static_cast<float>(eps);
  }
  if (nccl_transport_) {
    TORCH_CHECK(!interleave, "interleaved row ownership needs the peer-to-peer transport");
    cudaStream_t stream = current_stream();
    at::Tensor C = torch::empty({g.M, g.N}, A.options());
    engine_.gemm(g, C.data_ptr(), nullptr, nullptr, stream);
    if (norm.gamma != nullptr) {
      at::Tensor R = torch::empty_like(D);
      FO_NCCL_CHECK(ncclReduceScatter(C.data_ptr(), R.data_ptr(), R.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
      FO_CUDA_CHECK(launch_rmsnorm(R.data_ptr(), D.data_ptr(), norm.gamma, g.M / ws, g.N, norm.eps, g.dtype, stream));
    } else {
      FO_NCCL_CHECK(ncclReduceScatter(C.data_ptr(), D.data_ptr(), D.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
    }
    return;
  }
  engine_.gemm_reducescatter(g, D.data_ptr(), interleave, norm, nullptr, nullptr, current_stream());
}

void OverlapImpl::AllGatherGemm(at::Tensor A_shard, at::Tensor B, at::Tensor C, int64_t algo) {
  check_gemm_args(A_shard, B, nullptr);
  require_comm("allgather_gemm");
  TORCH_CHECK(engine_ready_, "allgather_gemm: call nccl_init first");
  TORCH_CHECK(algo >= 0 && algo < kNumAlgos, "Algo out of range");
  c10::cuda::CUDAGuard guard(A_shard.device());
  const int ws = comm_.world();
  const int64_t M = A_shard.size(0) * ws, N = B.size(0), K = A_shard.size(1);
  const TileConfig tc = algo_config(static_cast<int>(algo));
  TORCH_CHECK(M % tc.bm == 0 && N % tc.bn == 0 && K % 8 == 0, "need M % ", tc.bm, " == 0, N % ", tc.bn,
              " == 0, K % 8 == 0 (M = ", M, ", N = ", N, ", K = ", K, ")");
  check_matrix(C, "C");
  TORCH_CHECK(C.scalar_type() == A_shard.scalar_type() && C.size(0) == M && C.size(1) == N, "C must be [M, N]");
  if (nccl_transport_) {
    cudaStream_t stream = current_stream();
    at::Tensor full = torch::empty({M, K}, A_shard.options());
    FO_NCCL_CHECK(ncclAllGather(A_shard.data_ptr(), full.data_ptr(), A_shard.numel(), nccl_type(A_shard), comm_.get(),
                                stream));
    engine_.gemm(operands(full, B, algo), C.data_ptr(), nullptr, nullptr, stream);
    return;
  }
  engine_.allgather_gemm(A_shard.data_ptr(), B.data_ptr(), C.data_ptr(), static_cast<int>(M), static_cast<int>(N),
                         static_cast<int>(K), dtype_of(A_shard), static_cast<int>(algo), current_stream());
}

int64_t OverlapImpl::A2aPaddedRows(at::Tensor mLen_CPU, int64_t algo) {
  check_int_tensor(mLen_CPU, "mLen_CPU", false);
  const int ws = comm_.world();
  TORCH_CHECK(mLen_CPU.numel() == static_cast<int64_t>(ws) * ws, "mLen_CPU must be [size, size]");
  TORCH_CHECK(algo >= 0 && algo < kNumAlgos, "Algo out of range");
  return engine_.a2a_padded_rows(mLen_CPU.data_ptr<int>(), static_cast<int>(algo));
}

void OverlapImpl::A2aDispatchGemm(at::Tensor A_send, at::Tensor B, at::Tensor C, at::Tensor mLen_CPU, int64_t algo) {
  check_gemm_args(A_send, B, nullptr);
  require_comm("a2a_dispatch_gemm");
  TORCH_CHECK(engine_ready_, "a2a_dispatch_gemm: call nccl_init first");
  TORCH_CHECK(!nccl_transport_, "a2a_dispatch_gemm needs the peer-to-peer transport (all ranks on one node)");
  const int ws = comm_.world(), rank = comm_.rank();
  const int64_t m_pad = A2aPaddedRows(mLen_CPU, algo);
  const int* len = mLen_CPU.data_ptr<int>();
  int64_t send = 0;
  for (int j = 0; j < ws; ++j) {
    TORCH_CHECK(len[rank * ws + j] >= 0, "mLen_CPU entries must be >= 0");
    send += len[rank * ws + j];
  }
  TORCH_CHECK(A_send.size(0) >= send, "A_send has ", A_send.size(0), " rows but mLen_CPU sends ", send);
  const int64_t N = B.size(0), K = A_send.size(1);
  const TileConfig tc = algo_config(static_cast<int>(algo));
  TORCH_CHECK(N % tc.bn == 0 && K % 8 == 0, "need N % ", tc.bn, " == 0 and K % 8 == 0");
  check_matrix(C, "C");
  TORCH_CHECK(C.scalar_type() == A_send.scalar_type() && C.size(0) >= m_pad && C.size(1) == N,
              "C must be [>= ", m_pad, ", N]");
  c10::cuda::CUDAGuard guard(A_send.device());
  engine_.a2a_gemm(A_send.data_ptr(), B.data_ptr(), C.data_ptr(), len, static_cast<int>(N), static_cast<int>(K),
                   dtype_of(A_send), static_cast<int>(algo), current_stream());
}

void OverlapImpl::GemmRmsNorm(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor O, at::Tensor weight, double eps,
                              int64_t algo) {
  check_gemm_args(A, B, &C);
  c10::cuda::CUDAGuard guard(A.device());
  GemmOperands g = operands(A, B, algo);
  check_matrix(O, "O");
  TORCH_CHECK(O.scalar_type() == A.scalar_type() && O.numel() == C.numel(), "O must match C");
  TORCH_CHECK(weight.is_cuda() && weight.is_contiguous() && weight.numel() == g.N &&
                  weight.scalar_type() == A.scalar_type(),
              "weight must be a contiguous CUDA tensor of N values with A's dtype");
  NormArgs norm;
  norm.gamma = weight.data_ptr();
  norm.eps = static_cast<float>(eps);
  engine_.gemm_rmsnorm(g, C.data_ptr(), O.data_ptr(), norm, current_stream());
}

void OverlapImpl::AttachSymmetric(std::vector<int64_t> peer_ptrs, int64_t mc_ptr, int64_t nbytes) {
  TORCH_CHECK(engine_ready_, "attach_symmetric: call nccl_init first");
  TORCH_CHECK(static_cast<int>(peer_ptrs.size()) == comm_.world(), "attach_symmetric: need one pointer per rank");
  TORCH_CHECK(nbytes > 0, "attach_symmetric: nbytes must be positive");
  std::vector<void*> ptrs;
  for (int64_t v : peer_ptrs) ptrs.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(v)));
  engine_.attach_symmetric(static_cast<size_t>(nbytes), ptrs, reinterpret_cast<void*>(static_cast<uintptr_t>(mc_ptr)));
}
void OverlapImpl::DetachSymmetric() {
  TORCH_CHECK(engine_ready_, "detach_symmetric: call nccl_init first");
  engine_.detach_symmetric();
}
void OverlapImpl::SetUseNvls(bool allreduce, bool reducescatter) { engine_.set_use_nvls(allreduce, reducescatter); }
void OverlapImpl::SetAllGatherMulticast(bool on) { engine_.set_allgather_multicast(on); }
bool OverlapImpl::NvlsAvailable() { return engine_.nvls_available(); }
bool OverlapImpl::AllReduceUsesNvls() { return engine_.allreduce_uses_nvls(); }

void OverlapImpl::P2pPush(int64_t bytes, int64_t ctas) {
  require_comm("p2p_push");
  TORCH_CHECK(engine_ready_, "p2p_push: call nccl_init first");
  engine_.p2p_push(bytes, static_cast<int>(ctas), current_stream());
}

void OverlapImpl::P2pPushBulk(int64_t bytes, int64_t chunk_bytes, int64_t ctas) {
  require_comm("p2p_push_bulk");
  TORCH_CHECK(engine_ready_, "p2p_push_bulk: call nccl_init first");
  engine_.p2p_push_bulk(bytes, static_cast<int>(chunk_bytes), static_cast<int>(ctas), current_stream());
}

void OverlapImpl::MultimemBench(std::string kind, int64_t bytes, int64_t ctas, bool bf16) {
  require_comm("multimem_bench");
  TORCH_CHECK(engine_ready_, "multimem_bench: call nccl_init first");
  int k = -1;
  if (kind == "ld_reduce") k = MM_LD_REDUCE;
  else if (kind == "st") k = MM_ST;
  else if (kind == "allreduce") k = MM_ALLREDUCE;
  TORCH_CHECK(k >= 0, "multimem_bench: kind must be ld_reduce, st or allreduce");
  engine_.multimem_bench(k, bytes, static_cast<int>(ctas), bf16 ? DT_BF16 : DT_F16, current_stream());
}

void OverlapImpl::WaitOnUnsetCounter(int64_t timeout_ms) {
  TORCH_CHECK(timeout_ms > 0 && timeout_ms <= 5000, "timeout must be in (0, 5000] ms");
  engine_.wait_on_unset_counter(timeout_ms, current_stream());
}

void OverlapImpl::SetTransport(std::string name) {
  TORCH_CHECK(name == "p2p" || name == "nccl", "transport must be \"p2p\" or \"nccl\"");
  nccl_transport_ = name == "nccl" && comm_.world() > 1;
}
std::string OverlapImpl::Transport() { return nccl_transport_ ? "nccl" : "p2p"; }

void OverlapImpl::SetTimeoutMs(int64_t ms) {
  TORCH_CHECK(ms > 0, "timeout must be positive");
  engine_.set_timeout_ms(ms);
}
void OverlapImpl::SetSmCount(int64_t n) { engine_.set_sm_count(static_cast<int>(n)); }
void OverlapImpl::SetL2Hints(bool on) { engine_.set_l2_hints(on); }
void OverlapImpl::SetRasterTaper(bool on) { engine_.set_raster_taper(on); }
void OverlapImpl::SetRasterGroup(int64_t g) { engine_.set_raster_group(static_cast<int>(g)); }
void OverlapImpl::SetPhaseTrace(at::Tensor buf) {
  if (buf.numel() == 0) {
    engine_.set_phase_trace(nullptr);
    phase_trace_ = at::Tensor();
    return;
  }
  TORCH_CHECK(buf.is_cuda() && buf.is_contiguous() && buf.scalar_type() == at::kLong, "trace buffer must be a contiguous CUDA int64 tensor");
  TORCH_CHECK(buf.numel() >= kTraceWords * device_sm_count(), "trace buffer needs ", kTraceWords, " entries per SM (",
              kTraceWords * device_sm_count(), ")");
  phase_trace_ = buf;  // keeps the memory alive
  engine_.set_phase_trace(reinterpret_cast<unsigned long long*>(buf.data_ptr<int64_t>()));
}

void OverlapImpl::SetRowTrace(at::Tensor buf) {
  if (buf.numel() == 0) {
    engine_.set_row_trace(nullptr, 0);
    row_trace_ = at::Tensor();
    return;
  }
  TORCH_CHECK(buf.is_cuda() && buf.is_contiguous() && buf.scalar_type() == at::kLong && buf.numel() % 6 == 0,
              "row trace buffer must be a contiguous CUDA int64 tensor of 6 * rows entries");
  row_trace_ = buf;  // keeps the memory alive
  engine_.set_row_trace(reinterpret_cast<unsigned long long*>(buf.data_ptr<int64_t>()), buf.numel() / 6);
}

std::vector<int64_t> OverlapImpl::Status() {
  StatusWord s = engine_.read_status();
  return {s.code, s.rank, s.where, s.seen, s.want};
}
std::string OverlapImpl::StatusString() { return FusedEngine::describe(engine_.read_status()); }
void OverlapImpl::CheckStatus() {
  StatusWord s = engine_.read_status();
  TORCH_CHECK(s.code == ST_OK, "flashoverlap kernel reported a failure: ", FusedEngine::describe(s));
}
void OverlapImpl::Reset() { engine_.reset_counters(); }
int64_t OverlapImpl::NumAlgos() { return kNumAlgos; }
std::vector<int64_t> OverlapImpl::AlgoTile(int64_t algo) {
  TORCH_CHECK(algo >= 0 && algo < kNumAlgos, "Algo out of range");
  const TileConfig tc = algo_config(static_cast<int>(algo));
  return {tc.bm, tc.bn, tc.bk};
}

}  // namespace fo
