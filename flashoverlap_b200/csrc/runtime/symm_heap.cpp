#include "symm_heap.h"

#include <cstdint>
#include <cstring>
#include <stdexcept>

namespace fo {

std::string cuda_error_string(cudaError_t e, const char* what) {
  return std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
}

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(cuda_error_string(e, what));
}

SymmHeap::~SymmHeap() {
  try {
    destroy();
  } catch (...) {
  }
}

void SymmHeap::init(int rank, int world, size_t bytes, const AllGatherFn& all_gather) {
  if (valid()) throw std::runtime_error("SymmHeap::init called twice");
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("SymmHeap::init: bad rank/world");
  const size_t gran = size_t(2) << 20;
  bytes = (bytes + gran - 1) / gran * gran;
  rank_ = rank;
  world_ = world;
  bytes_ = bytes;
  top_ = 0;
  check(cudaMalloc(&base_, bytes), "cudaMalloc(symmetric slab)");
  check(cudaMemset(base_, 0, bytes), "cudaMemset(symmetric slab)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  peer_base_.assign(world, nullptr);
  peer_base_[rank] = base_;
  if (world == 1) return;
  if (!all_gather) throw std::runtime_error("SymmHeap::init: world > 1 needs an all_gather callback");

  cudaIpcMemHandle_t mine;
  check(cudaIpcGetMemHandle(&mine, base_), "cudaIpcGetMemHandle");
  std::vector<cudaIpcMemHandle_t> all(world);
  all_gather(&mine, sizeof(mine), all.data());
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    void* p = nullptr;
    check(cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    peer_base_[r] = p;
  }
  // A second exchange doubles as a barrier: nobody proceeds (and possibly
  // writes into a peer) before every rank has zeroed and mapped its slab.
  char token = 1;
  std::vector<char> tokens(world);
  all_gather(&token, 1, tokens.data());
}

void SymmHeap::attach(int rank, int world, size_t bytes, const std::vector<void*>& peer_ptrs, void* mc_ptr) {
  if (valid()) throw std::runtime_error("SymmHeap::attach: heap already initialised");
  if (world < 1 || rank < 0 || rank >= world || static_cast<int>(peer_ptrs.size()) != world) {
    throw std::runtime_error("SymmHeap::attach: bad rank / world / pointer list");
  }
  for (void* p : peer_ptrs) {
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 1023u)) {
      throw std::runtime_error("SymmHeap::attach: peer pointers must be non-null and 1024-byte aligned");
    }
  }
  rank_ = rank;
  world_ = world;
  bytes_ = bytes;
  top_ = 0;
  peer_base_ = peer_ptrs;
  base_ = peer_ptrs[rank];
  mc_base_ = mc_ptr;
  owned_ = false;
}

void SymmHeap::destroy() {
  if (!valid()) return;
  if (!owned_) {
    peer_base_.clear();
    base_ = mc_base_ = nullptr;
    bytes_ = top_ = 0;
    owned_ = true;
    return;
  }
  for (int r = 0; r < world_; ++r) {
    if (r != rank_ && peer_base_[r] != nullptr) cudaIpcCloseMemHandle(peer_base_[r]);
  }
  peer_base_.clear();
  cudaFree(base_);
  base_ = nullptr;
  bytes_ = top_ = 0;
}

size_t SymmHeap::alloc(size_t bytes, size_t align) {
  if (!valid()) throw std::runtime_error("SymmHeap::alloc before init");
  size_t off = (top_ + align - 1) / align * align;
  if (off + bytes > bytes_) throw std::runtime_error("SymmHeap: out of symmetric memory");
  top_ = off + bytes;
  return off;
}

bool SymmHeap::contains_local(const void* p, size_t bytes) const {
  const char* c = static_cast<const char*>(p);
  const char* b = static_cast<const char*>(base_);
  return valid() && c >= b && c + bytes <= b + bytes_;
}

}  // namespace fo
