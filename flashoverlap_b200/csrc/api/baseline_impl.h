// torch.classes.flashoverlap_class.BaselineImpl: the non-overlapped baseline,
// a cuBLAS GEMM followed by one NCCL collective on the same stream
// (reference: src/baseline_impl.{h,cu}).  fp32 accumulation is used for both
// 16-bit types.  Unlike the reference (src/baseline_impl.cu:38-40), a single
// rank still computes the GEMM.
#pragma once

#include <cublas_v2.h>
#include <torch/custom_class.h>
#include <torch/torch.h>

#include "nccl_utils.h"

namespace fo {

class BaselineImpl : public torch::CustomClassHolder {
 public:
  BaselineImpl();
  ~BaselineImpl() override;

  void NcclInit(int64_t rank, int64_t size, std::vector<int64_t> id);
  void CublasInit();
  void GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C);
  void GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D);
  void GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor mLen_CPU);
  void Gemm(at::Tensor A, at::Tensor B, at::Tensor C);
  void NcclAllReduce(at::Tensor C);
  void NcclReduceScatter(at::Tensor C);
  void NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU);

 private:
  void gemm_on(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, cudaStream_t stream);
  void all2all(const at::Tensor& C, at::Tensor& D, const at::Tensor& mLen, int64_t width, cudaStream_t stream);
  Communicator comm_;
  cublasHandle_t handle_ = nullptr;
  void* workspace_ = nullptr;
  size_t workspace_bytes_ = 0;
};

}  // namespace fo
