// NCCL bootstrap helpers shared by the two implementation classes
// (reference: src/mccl_utils.{h,cpp}, src/nccl_utils.{h,cu}).  Errors throw
// instead of terminating the process, and communicators are destroyed with
// their owner.
#pragma once

#include <nccl.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace fo {

#define FO_NCCL_CHECK(cmd)                                                                            \
  do {                                                                                                \
    ncclResult_t r_ = (cmd);                                                                          \
    if (r_ != ncclSuccess) {                                                                          \
      throw std::runtime_error(std::string("NCCL failure ") + ncclGetErrorString(r_) + " at " +      \
                               __FILE__ + ":" + std::to_string(__LINE__));                           \
    }                                                                                                 \
  } while (0)

#define FO_CUDA_CHECK(cmd)                                                                            \
  do {                                                                                                \
    cudaError_t e_ = (cmd);                                                                           \
    if (e_ != cudaSuccess) {                                                                          \
      throw std::runtime_error(std::string("CUDA failure ") + cudaGetErrorString(e_) + " at " +      \
                               __FILE__ + ":" + std::to_string(__LINE__));                           \
    }                                                                                                 \
  } while (0)

constexpr int kUniqueIdWords = NCCL_UNIQUE_ID_BYTES / 8;  // 16 x int64

// A fresh NCCL unique id as 16 int64 words (rank 0 calls this and broadcasts).
std::vector<int64_t> generate_nccl_id();
ncclUniqueId id_from_words(const std::vector<int64_t>& words);

// RAII communicator.  world == 1 keeps no communicator (like the reference,
// which stores a null communicator for a single rank).
class Communicator {
 public:
  Communicator() = default;
  ~Communicator();
  Communicator(const Communicator&) = delete;
  Communicator& operator=(const Communicator&) = delete;
  void init(int rank, int world, const std::vector<int64_t>& id_words);
  ncclComm_t get() const { return comm_; }
  bool active() const { return comm_ != nullptr; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  // Host-to-host all-gather through the communicator (small control data).
  void all_gather_host(const void* send, size_t bytes, void* recv) const;

 private:
  ncclComm_t comm_ = nullptr;
  int rank_ = 0, world_ = 1;
};

}  // namespace fo
