// FusedEngine: host-side orchestration of the fused sm_100a kernel.
//
// Owns the symmetric workspace (staging buffers for partial results, result
// buffers for all-reduce, arrival counters), the device status word and the
// per-call bookkeeping (which of the two staging/counter sets a call uses).
// It plays the role of the reference's OverlapImpl host code
// (reference: src/overlap_impl.cu:221-328) but issues exactly one kernel per
// operation: no second stream, no wait kernels, no NCCL calls.
//
// Why two sets of staging buffers and counters are enough: a rank can finish
// call i only after every rank has pushed its share of call i, hence after
// every rank has finished call i-1.  A rank can therefore run at most one call
// ahead of any other, so the set used by call i-1 is quiet when call i+1
// starts, and the counters of the set used by call i+1 can be cleared by a
// memset that is ordered on the stream before call i.
#pragma once

#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../kernels/fused_params.h"
#include "../kernels/comm_kernels.h"
#include "../kernels/gemm_launch.h"
#include "symm_heap.h"

namespace fo {

struct NormArgs {
  const void* gamma = nullptr;  // null = no RMSNorm
  float eps = 1e-5f;
};

// Reference-compatible signalling for the plain GEMM (see FusedParams).
struct SignalArgs {
  int* seg_counter = nullptr;
  const int* cseg = nullptr;
  int nseg = 0;
  int* ticket_counter = nullptr;
  int* trace = nullptr;
  const int* slot_of_tile = nullptr;
};

class FusedEngine {
 public:
  static constexpr int kMaxTileRows = fo::kMaxTileRows;

  FusedEngine() = default;
  ~FusedEngine();

  void init(int rank, int world, AllGatherFn all_gather);
  bool initialized() const { return status_dev_ != nullptr; }
  int rank() const { return rank_; }
  int world() const { return world_; }

  void set_timeout_ms(long long ms) { timeout_ns_ = static_cast<unsigned long long>(ms) * 1000000ull; }
  void set_sm_count(int n) { sm_count_ = n; }
  void set_raster_group(int g) { raster_group_ = g; }
  // L2 eviction hints on the operand loads (A row panel kept, B streamed); off by default
  // (they help only the largest K, measured).
  void set_l2_hints(bool on) { l2_hints_ = on; }
  // Shrinking last raster groups for operations with a reduce phase (default on).
  void set_raster_taper(bool on) { raster_taper_ = on; }
  // Device buffer of kTraceWords x uint64 per CTA that every following launch
  // fills with its phase timestamps (null = off).
  void set_phase_trace(unsigned long long* buf) { phase_trace_ = buf; }
  // Device buffer of `rows` x 6 x uint64: the reduce phase of every following
  // launch of at most `rows` rows records, per global row, when it was claimed,
  // ready, summed, past its barrier and stored, and which CTA and row group did it (null = off).
  void set_row_trace(unsigned long long* buf, long long rows) {
    row_trace_ = buf;
    row_trace_rows_ = buf != nullptr ? rows : 0;
  }

  // C[M,N] = A[M,K] * B[N,K]^T on this GPU only.  `layout` null = row-major.
  void gemm(const GemmOperands& g, void* C, const OutLayout* layout, const SignalArgs* sig, cudaStream_t stream);

  // GEMM + RMSNorm on one GPU (world size 1 form of the fused operations):
  // `scratch` receives the un-normalised product, `out` the normalised rows.
  void gemm_rmsnorm(const GemmOperands& g, void* scratch, void* out, const NormArgs& norm, cudaStream_t stream);

  // Fused GEMM + all-reduce (+ RMSNorm).  Collective: every rank of the group
  // must call it with the same shapes.  The result lands in a symmetric result
  // buffer whose address is returned; if `out_user` is not null the result is
  // also copied there (stream-ordered).  The returned buffer stays valid until
  // the second next fused call on this engine.
  void* gemm_allreduce(const GemmOperands& g, void* out_user, const NormArgs& norm, const OutLayout* out_layout,
                       const SignalArgs* sig, cudaStream_t stream);

  // Fused GEMM + reduce-scatter (+ RMSNorm) into D [M/world, N] (local memory).
  // interleave = false: rank r receives rows [r*M/world, (r+1)*M/world).
  // interleave = true : rank r receives rows r, r+world, r+2*world, ... (the
  // ownership of the reference's scatter epilogue, reference:
  // src/overlap/gemm_with_scatter.h:161-177, example/utils.py:24-52).
  void gemm_reducescatter(const GemmOperands& g, void* D, bool interleave, const NormArgs& norm,
                          const OutLayout* out_layout, const SignalArgs* sig, cudaStream_t stream);

  // Fused all-gather + GEMM (column-parallel linear on sequence-sharded
  // activations): C[M, N] = gather_r(A_r)[M, K] * B[N, K]^T where every rank
  // holds A_r = rows [r*M/world, (r+1)*M/world).  One launch: spare warps push
  // this rank's shard to all ranks while the tensor cores start on it; tiles of
  // other shards wait (bounded) for that shard's counter.  Collective.
  void allgather_gemm(const void* A_shard, const void* B, void* C, int M, int N, int K, DType dtype, int algo,
                      cudaStream_t stream);

  // Fused all-to-all dispatch + GEMM (tokens routed to the rank that holds
  // their expert): rank i sends rows_to[j] = mlen[i*world + j] rows of A_send
  // (packed in destination order, its own block included) to rank j; every rank
  // then multiplies the rows it received (in source order) by its B:
  // C[0 .. received) = recv[received, K] * B[N, K]^T.  C must have room for
  // `padded_rows(mlen)` rows (the largest receive count over all ranks, rounded
  // up to the tile height); rows past `received` are scratch.  One launch,
  // same mechanism as allgather_gemm.  Collective; `mlen` is the full world x
  // world matrix and must be identical on all ranks.
  void a2a_gemm(const void* A_send, const void* B, void* C, const int* mlen, int N, int K, DType dtype, int algo,
                cudaStream_t stream);
  // Rows of the gathered buffer / of C needed by a2a_gemm for this matrix and Algo.
  int a2a_padded_rows(const int* mlen, int algo) const;

  // Collective bandwidth primitive: every rank stores `bytes` to each of the
  // other ranks with the push kernel and then waits, on the device, until the
  // pushes of all peers have landed here.  Used by the bandwidth-curve tool.
  void p2p_push(long long bytes, int ctas, cudaStream_t stream);
  // Same transfer with bulk copies out of shared memory (`chunk_bytes` per copy).
  void p2p_push_bulk(long long bytes, int chunk_bytes, int ctas, cudaStream_t stream);
  // Collective NVLink SHARP primitive over `bytes` of symmetric memory (needs a
  // multicast mapping): kind MM_LD_REDUCE / MM_ST / MM_ALLREDUCE, every rank
  // handles its 1/world share, then waits until all ranks are done.
  void multimem_bench(int kind, long long bytes, int ctas, DType dtype, cudaStream_t stream);

  // Collective.  Hands the engine externally allocated symmetric memory (see
  // SymmHeap::attach) to carve its workspace from; with a multicast mapping
  // the fused operations switch to the NVLink SHARP path.  The memory is
  // zero-filled here and must outlive the engine.
  void attach_symmetric(size_t bytes, const std::vector<void*>& peer_ptrs, void* mc_ptr);
  // Collective.  Gives attached memory back (after draining the device): the
  // next fused call allocates the engine's own peer-mapped heap.
  void detach_symmetric();
  bool nvls_available() const { return heap_.valid() && heap_.has_multicast() && world_ > 1; }
  // Which operations take the NVLink SHARP path when it is available.
  // Default: none.  For an output of S bytes an all-reduce moves S(1+1/n)
  // bytes per NVLink direction through the switch against 2S(n-1)/n with
  // peer-to-peer stores (fewer from four ranks on), but half of the
  // peer-to-peer traffic, the partial tiles, leaves from the GEMM's epilogue
  // while the GEMM runs, and the switch can only pull complete rows: measured
  // with 4 and 8 ranks the peer-to-peer form is the faster one.  A
  // reduce-scatter moves S(n-1)/n with peer-to-peer pushes against S pulled
  // through the switch.  set_use_nvls fixes both choices by hand,
  // set_nvls_auto_min_world makes the all-reduce switch over by group size.
  void set_use_nvls(bool allreduce, bool reducescatter) {
    nvls_ar_ = allreduce ? 1 : 0;
    nvls_rs_ = reducescatter ? 1 : 0;
  }
  // All-gather -> GEMM: push the shard with one multicast store per chunk (off by default, see nvls_ag_).
  void set_allgather_multicast(bool on) { nvls_ag_ = on; }
  bool allreduce_uses_nvls() const {
    return nvls_available() && (nvls_ar_ < 0 ? nvls_auto_min_world_ > 0 && world_ >= nvls_auto_min_world_ : nvls_ar_ != 0);
  }
  // Smallest group for which the all-reduce takes NVLink SHARP by itself (0 = never).
  void set_nvls_auto_min_world(int n) { nvls_auto_min_world_ = n; }
  bool reducescatter_uses_nvls() const { return nvls_available() && nvls_rs_ > 0; }

  // Failure-path self test: launches the bounded counter wait on a counter that
  // nothing increments, with its own short deadline.  The wait must give up,
  // record ST_TIMEOUT_FLAG in the status word and leave the context usable.
  void wait_on_unset_counter(long long timeout_ms, cudaStream_t stream);

  // Collective.  Makes sure the symmetric workspace can hold an M x N problem.
  void ensure_workspace(long long m, long long n);

  // Throws if a kernel launched earlier by this engine has reported a failure
  // (reads the host mirror of the status word; no synchronisation).  Every
  // operation calls it first, so a timed-out wait cannot pass unnoticed.
  void check_previous(const char* op) const;

  // Reads the device status word (synchronises the device).  code == ST_OK
  // means no kernel has reported a failure since the last clear.
  StatusWord read_status();
  void clear_status();
  // Collective; after a failed call: waits for the device, zeroes all counters.
  void reset_counters();

  static std::string describe(const StatusWord& s);

 private:
  struct Workspace {
    size_t stage[2] = {0, 0};
    size_t result[2] = {0, 0};
    size_t flags[2] = {0, 0};  // kMaxTileRows arrival counters + 1 delivery counter each
    size_t misc = 0;           // counters that the per-call clearing must not touch
    size_t local_flags = 0;    // arrival counters of single-GPU operations (never written by peers)
    long long capacity_elems = 0;
  };
  void base_params(FusedParams& p, const SignalArgs* sig);
  uint32_t* flag_ptr(int rank, int set) const;
  uint32_t* done_ptr(int rank, int set) const;

  int rank_ = 0, world_ = 1;
  AllGatherFn all_gather_;
  SymmHeap heap_;
  Workspace ws_;
  StatusWord* status_dev_ = nullptr;
  StatusWord* status_host_ = nullptr;    // mirror of the status word in mapped host memory (host address)
  StatusWord* status_mirror_ = nullptr;  // the same memory as the device sees it
  unsigned long long timeout_ns_ = 20000000000ull;
  int sm_count_ = 0;
  int raster_group_ = 0;  // 0 = choose per operation
  bool l2_hints_ = false;
  bool raster_taper_ = true;
  int nvls_ar_ = -1;  // -1 = by group size, 0 = off, 1 = on
  int nvls_auto_min_world_ = 0;
  int nvls_rs_ = -1;
  void carve_workspace(long long elems);
  static constexpr size_t kNoMulticast = ~size_t(0);
  void gathered_gemm(const void* const* src_for, const long long* bytes_for, const int* src_end, int M, int first_row,
                     const void* B, void* C, int N, int K, DType dtype, int algo, const char* op, cudaStream_t stream,
                     size_t mc_slot_offset, const void* a_own, int own_rows);
  // All-gather pushes through the switch (one multimem.st per chunk) deliver every shard at the same time,
  // at the end; the ring of peer-to-peer stores delivers one shard per step in the order the GEMM consumes
  // them, which is what lets the GEMM overlap the transfer: multicast is an option, not the default.
  bool nvls_ag_ = false;
  unsigned long long* phase_trace_ = nullptr;
  unsigned long long* row_trace_ = nullptr;
  long long row_trace_rows_ = 0;
  unsigned long long calls_ = 0;  // fused collective calls issued so far
  void* ag_dst_scratch_[kMaxRanks] = {};  // destination of this rank's block on every rank (per call)
  unsigned long long pushes_ = 0;  // arrivals expected at the push counter so far
  unsigned long long mm_arrivals_ = 0;  // arrivals expected at the multimem benchmark counter so far
  void push_common(long long bytes, int chunk_bytes, int ctas, cudaStream_t stream);
};

}  // namespace fo
