// Argument validation shared by the torch-facing classes.  The reference does
// none (a wrong cSeg sum makes its wait kernel spin forever, reference:
// src/wait.cuh:5-9); here every entry point checks before launching.
#pragma once

#include <torch/torch.h>

#include <vector>

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

// Index arrays that a kernel stores through are validated on the host before
// the launch: a stale or corrupt tuning file must not become a write outside a
// buffer (possibly a peer GPU's).  The check costs a device synchronisation,
// so its outcome is remembered per (storage address, tensor version, length):
// the same tensor object is checked again only after it has been written.
class IndexCheckCache {
 public:
  // `t` must hold every value of [0, n) exactly once (a tile-to-slot map).
  void require_permutation(const at::Tensor& t, int64_t n, const char* name) {
    if (seen(t, n, 0)) return;
    TORCH_CHECK(t.numel() == n, name, " must have ", n, " entries, has ", t.numel());
    if (n > 0) {
      auto flat = t.reshape({-1}).to(at::kLong);
      const int64_t lo = flat.min().item<int64_t>(), hi = flat.max().item<int64_t>();
      TORCH_CHECK(lo >= 0 && hi < n, name, " holds ", lo < 0 ? lo : hi, ", outside [0, ", n, ")");
      TORCH_CHECK(at::bincount(flat, {}, n).max().item<int64_t>() == 1, name, " is not a permutation of 0..", n - 1,
                  ": some slot appears twice");
    }
    remember(t, n, 0);
  }
  // every value of `t` must lie in [0, limit)
  void require_range(const at::Tensor& t, int64_t limit, const char* name) {
    if (seen(t, limit, 1)) return;
    if (t.numel() > 0) {
      const int64_t lo = t.min().item<int64_t>(), hi = t.max().item<int64_t>();
      TORCH_CHECK(lo >= 0 && hi < limit, name, " holds ", lo < 0 ? lo : hi, ", outside [0, ", limit, ")");
    }
    remember(t, limit, 1);
  }

 private:
  struct Key {
    const void* ptr;
    uint32_t version;
    int64_t numel, bound;
    int kind;
    bool operator==(const Key& o) const {
      return ptr == o.ptr && version == o.version && numel == o.numel && bound == o.bound && kind == o.kind;
    }
  };
  static Key key_of(const at::Tensor& t, int64_t bound, int kind) {
    return Key{t.data_ptr(), static_cast<uint32_t>(t._version()), t.numel(), bound, kind};
  }
  bool seen(const at::Tensor& t, int64_t bound, int kind) const {
    const Key k = key_of(t, bound, kind);
    for (const Key& e : entries_) {
      if (e == k) return true;
    }
    return false;
  }
  void remember(const at::Tensor& t, int64_t bound, int kind) {
    if (entries_.size() >= 16) entries_.erase(entries_.begin());
    entries_.push_back(key_of(t, bound, kind));
  }
  std::vector<Key> entries_;
};

}  // namespace fo
