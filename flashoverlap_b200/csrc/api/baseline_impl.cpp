#include "baseline_impl.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "checks.h"

namespace fo {

namespace {
ncclDataType_t nccl_type(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16 ? ncclBfloat16 : ncclHalf; }
cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void cublas_check(cublasStatus_t s, const char* what) {
  TORCH_CHECK(s == CUBLAS_STATUS_SUCCESS, what, " failed with cuBLAS status ", static_cast<int>(s));
}
}  // namespace

BaselineImpl::BaselineImpl() = default;

BaselineImpl::~BaselineImpl() {
  if (handle_ != nullptr) cublasDestroy(handle_);
  if (workspace_ != nullptr) cudaFree(workspace_);
}

void BaselineImpl::NcclInit(int64_t rank, int64_t size, std::vector<int64_t> id) {
  comm_.init(static_cast<int>(rank), static_cast<int>(size), id);
}

void BaselineImpl::CublasInit() {
  if (handle_ == nullptr) {
    cublas_check(cublasCreate(&handle_), "cublasCreate");
    // A fixed workspace keeps cuBLAS from allocating inside the timed region.
    workspace_bytes_ = size_t(64) << 20;
    FO_CUDA_CHECK(cudaMalloc(&workspace_, workspace_bytes_));
    cublas_check(cublasSetWorkspace(handle_, workspace_, workspace_bytes_), "cublasSetWorkspace");
  }
}

void BaselineImpl::gemm_on(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, cudaStream_t stream) {
  TORCH_CHECK(handle_ != nullptr, "call cublas_init first");
  check_gemm_args(A, B, &C);
  const int M = static_cast<int>(A.size(0)), N = static_cast<int>(B.size(0)), K = static_cast<int>(A.size(1));
  const cudaDataType_t dt = A.scalar_type() == at::kBFloat16 ? CUDA_R_16BF : CUDA_R_16F;
  const float alpha = 1.f, beta = 0.f;
  cublas_check(cublasSetStream(handle_, stream), "cublasSetStream");
  // Row-major C[M,N] = A[M,K] * B[N,K]^T is column-major C^T[N,M] = B^T-as-stored (op T) * A-as-stored (op N).
  cublas_check(cublasGemmEx(handle_, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, B.data_ptr(), dt, K, A.data_ptr(), dt,
                            K, &beta, C.data_ptr(), dt, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT),
               "cublasGemmEx");
}

void BaselineImpl::Gemm(at::Tensor A, at::Tensor B, at::Tensor C) {
  c10::cuda::CUDAGuard guard(A.device());
  gemm_on(A, B, C, current_stream());
}

void BaselineImpl::GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C) {
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = current_stream();
  gemm_on(A, B, C, stream);
  if (comm_.active()) {
    FO_NCCL_CHECK(ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
  }
}

void BaselineImpl::GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D) {
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = current_stream();
  gemm_on(A, B, C, stream);
  const int ws = comm_.world();
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && D.scalar_type() == C.scalar_type() && D.numel() * ws == C.numel(),
              "D must hold M*N/size elements of C's dtype");
  if (comm_.active()) {
    FO_NCCL_CHECK(ncclReduceScatter(C.data_ptr(), D.data_ptr(), D.numel(), nccl_type(C), ncclSum, comm_.get(), stream));
  } else {
    FO_CUDA_CHECK(cudaMemcpyAsync(D.data_ptr(), C.data_ptr(), C.nbytes(), cudaMemcpyDeviceToDevice, stream));
  }
}

void BaselineImpl::all2all(const at::Tensor& C, at::Tensor& D, const at::Tensor& mLen, int64_t width,
                           cudaStream_t stream) {
  const int ws = comm_.world(), rank = comm_.rank();
  check_int_tensor(mLen, "mLen_CPU", false);
  TORCH_CHECK(mLen.numel() == static_cast<int64_t>(ws) * ws, "mLen_CPU must be [size, size]");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous() && D.scalar_type() == C.scalar_type(), "D must match C's dtype");
  const int* len = mLen.data_ptr<int>();
  int64_t send_rows = 0, recv_rows = 0;
  for (int peer = 0; peer < ws; ++peer) {
    if (peer == rank) continue;
    TORCH_CHECK(len[rank * ws + peer] >= 0 && len[peer * ws + rank] >= 0, "mLen_CPU entries must be >= 0");
    send_rows += len[rank * ws + peer];
    recv_rows += len[peer * ws + rank];
  }
  TORCH_CHECK(send_rows * width <= C.numel() && recv_rows * width <= D.numel(), "mLen_CPU exceeds the buffers");
  if (!comm_.active()) return;
  const size_t esz = C.element_size();
  char* src = static_cast<char*>(C.data_ptr());
  char* dst = static_cast<char*>(D.data_ptr());
  FO_NCCL_CHECK(ncclGroupStart());
  for (int peer = 0; peer < ws; ++peer) {
    if (peer == rank) continue;
    const size_t n_send = static_cast<size_t>(len[rank * ws + peer]) * width;
    const size_t n_recv = static_cast<size_t>(len[peer * ws + rank]) * width;
    FO_NCCL_CHECK(ncclSend(src, n_send, nccl_type(C), peer, comm_.get(), stream));
    FO_NCCL_CHECK(ncclRecv(dst, n_recv, nccl_type(C), peer, comm_.get(), stream));
    src += n_send * esz;
    dst += n_recv * esz;
  }
  FO_NCCL_CHECK(ncclGroupEnd());
}

void BaselineImpl::GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor mLen_CPU) {
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = current_stream();
  gemm_on(A, B, C, stream);
  all2all(C, D, mLen_CPU, B.size(0), stream);
}

void BaselineImpl::NcclAllReduce(at::Tensor C) {
  TORCH_CHECK(C.is_cuda() && C.is_contiguous(), "C must be a contiguous CUDA tensor");
  dtype_of(C);
  c10::cuda::CUDAGuard guard(C.device());
  if (!comm_.active()) return;
  FO_NCCL_CHECK(
      ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_type(C), ncclSum, comm_.get(), current_stream()));
}

void BaselineImpl::NcclReduceScatter(at::Tensor C) {
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

void BaselineImpl::NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU) {
  TORCH_CHECK(C.is_cuda() && C.is_contiguous() && C.dim() == 2, "C must be a contiguous 2-D CUDA tensor");
  dtype_of(C);
  c10::cuda::CUDAGuard guard(C.device());
  all2all(C, D, mLen_CPU, C.size(1), current_stream());
}

}  // namespace fo
