#include "nccl_utils.h"

#include <cuda_runtime.h>

#include <cstring>

namespace fo {

std::vector<int64_t> generate_nccl_id() {
  ncclUniqueId id;
  FO_NCCL_CHECK(ncclGetUniqueId(&id));
  std::vector<int64_t> words(kUniqueIdWords);
  std::memcpy(words.data(), &id, NCCL_UNIQUE_ID_BYTES);
  return words;
}

ncclUniqueId id_from_words(const std::vector<int64_t>& words) {
  if (static_cast<int>(words.size()) != kUniqueIdWords) {
    throw std::runtime_error("NCCL id must have " + std::to_string(kUniqueIdWords) + " int64 entries, got " +
                             std::to_string(words.size()));
  }
  ncclUniqueId id;
  std::memcpy(&id, words.data(), NCCL_UNIQUE_ID_BYTES);
  return id;
}

Communicator::~Communicator() {
  if (comm_ != nullptr) ncclCommDestroy(comm_);
  comm_ = nullptr;
}

void Communicator::init(int rank, int world, const std::vector<int64_t>& id_words) {
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("nccl_init: bad rank / size");
  if (comm_ != nullptr) {
    ncclCommDestroy(comm_);
    comm_ = nullptr;
  }
  rank_ = rank;
  world_ = world;
  if (world == 1) return;
  ncclUniqueId id = id_from_words(id_words);
  FO_NCCL_CHECK(ncclCommInitRank(&comm_, world, id, rank));
}

void Communicator::all_gather_host(const void* send, size_t bytes, void* recv) const {
  if (world_ == 1) {
    std::memcpy(recv, send, bytes);
    return;
  }
  if (comm_ == nullptr) throw std::runtime_error("all_gather_host: communicator not initialised");
  void* d_send = nullptr;
  void* d_recv = nullptr;
  cudaStream_t s = nullptr;
  FO_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  FO_CUDA_CHECK(cudaMalloc(&d_send, bytes));
  FO_CUDA_CHECK(cudaMalloc(&d_recv, bytes * world_));
  FO_CUDA_CHECK(cudaMemcpyAsync(d_send, send, bytes, cudaMemcpyHostToDevice, s));
  FO_NCCL_CHECK(ncclAllGather(d_send, d_recv, bytes, ncclChar, comm_, s));
  FO_CUDA_CHECK(cudaMemcpyAsync(recv, d_recv, bytes * world_, cudaMemcpyDeviceToHost, s));
  FO_CUDA_CHECK(cudaStreamSynchronize(s));
  cudaFree(d_send);
  cudaFree(d_recv);
  cudaStreamDestroy(s);
}

}  // namespace fo
