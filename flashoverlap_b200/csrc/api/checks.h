// Argument validation shared by the torch-facing classes.  The reference does
// none (a wrong cSeg sum makes its wait kernel spin forever, reference:
// src/wait.cuh:5-9); here every entry point checks before launching.
#pragma once

#include <torch/torch.h>

#include "../kernels/gemm_launch.h"

namespace fo {

inline DType dtype_of(const at::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kHalf || t.scalar_type() == at::kBFloat16,
              "flashoverlap: tensors must be float16 or bfloat16, got ", t.scalar_type());
  return t.scalar_type() == at::kBFloat16 ? DT_BF16 : DT_F16;
}

inline void check_matrix(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.dim() == 2, name, " must be 2-D, got ", t.dim(), "-D");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous (row-major)");
}

inline void check_gemm_args(const at::Tensor& A, const at::Tensor& B, const at::Tensor* C) {
  check_matrix(A, "A");
  check_matrix(B, "B");
  TORCH_CHECK(A.scalar_type() == B.scalar_type(), "A and B must have the same dtype");
  dtype_of(A);
  TORCH_CHECK(A.size(1) == B.size(1), "A is [M,K] and B is [N,K]: K differs (", A.size(1), " vs ", B.size(1), ")");
  TORCH_CHECK(A.device() == B.device(), "A and B must be on the same device");
  if (C != nullptr) {
    check_matrix(*C, "C");
    TORCH_CHECK(C->scalar_type() == A.scalar_type(), "C must have the dtype of A");
    TORCH_CHECK(C->numel() == A.size(0) * B.size(0), "C must hold M*N = ", A.size(0) * B.size(0), " elements, has ",
                C->numel());
    TORCH_CHECK(C->device() == A.device(), "C must be on the device of A");
  }
}

inline void check_int_tensor(const at::Tensor& t, const char* name, bool cuda) {
  TORCH_CHECK(t.scalar_type() == at::kInt, name, " must be int32");
  TORCH_CHECK(t.is_cuda() == cuda, name, cuda ? " must be a CUDA tensor" : " must be a CPU tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

}  // namespace fo
