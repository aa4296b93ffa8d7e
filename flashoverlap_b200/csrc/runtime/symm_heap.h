// Symmetric peer-mapped memory for the fused kernels.
//
// Every rank allocates one slab of the same size with cudaMalloc, exports it
// as a CUDA IPC handle and maps the slabs of all peers, so that an offset into
// the slab names the same object on every GPU and `ptr(rank, offset)` can be
// stored to or loaded from by kernels on this GPU over NVLink.  The reference
// has no such object: it hands contiguous segments to NCCL instead
// (reference: src/overlap_impl.cu:257-265).
//
// Handle exchange is a callback so that the heap itself depends on nothing but
// the CUDA runtime (the torch classes exchange through their NCCL
// communicator; tests on one GPU use world size 1, which needs no exchange).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <functional>
#include <string>
#include <vector>

namespace fo {

// all_gather(send, bytes, recv): gathers `bytes` bytes from every rank into
// recv[rank * bytes ...]; host memory on both sides; collective over the group.
using AllGatherFn = std::function<void(const void* send, size_t bytes, void* recv)>;

class SymmHeap {
 public:
  SymmHeap() = default;
  ~SymmHeap();
  SymmHeap(const SymmHeap&) = delete;
  SymmHeap& operator=(const SymmHeap&) = delete;

  // Collective.  Allocates `bytes` (rounded up to 2 MiB) on the current device,
  // zero-fills it and maps every peer's slab.
  void init(int rank, int world, size_t bytes, const AllGatherFn& all_gather);
  // Adopts symmetric memory that somebody else allocated and mapped (for
  // example torch.distributed._symmetric_memory): peer_ptrs[r] is rank r's slab
  // as mapped into this process, mc_ptr the multicast (NVLink SHARP) mapping of
  // all slabs or null.  The heap does not own the memory.
  void attach(int rank, int world, size_t bytes, const std::vector<void*>& peer_ptrs, void* mc_ptr);
  // Unmaps peers and frees the slab.  The caller must make sure that no rank
  // still has kernels in flight that touch this heap.
  void destroy();

  bool valid() const { return base_ != nullptr; }
  size_t size() const { return bytes_; }
  int rank() const { return rank_; }
  int world() const { return world_; }

  // Bump allocation; identical call sequences on all ranks give identical
  // offsets.  Returns the offset; throws std::runtime_error when full.
  size_t alloc(size_t bytes, size_t align = 256);
  void reset_allocator() { top_ = 0; }
  size_t used() const { return top_; }

  void* ptr(int rank, size_t offset) const { return static_cast<char*>(peer_base_[rank]) + offset; }
  void* local(size_t offset) const { return static_cast<char*>(base_) + offset; }
  // Multicast address of `offset` (null when the heap has no multicast mapping).
  void* mc(size_t offset) const { return mc_base_ ? static_cast<char*>(mc_base_) + offset : nullptr; }
  bool has_multicast() const { return mc_base_ != nullptr; }
  bool owned() const { return owned_; }
  bool contains_local(const void* p, size_t bytes) const;

 private:
  int rank_ = 0, world_ = 1;
  size_t bytes_ = 0, top_ = 0;
  void* base_ = nullptr;
  void* mc_base_ = nullptr;
  bool owned_ = true;
  std::vector<void*> peer_base_;
};

std::string cuda_error_string(cudaError_t e, const char* what);

}  // namespace fo
