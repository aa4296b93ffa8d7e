// torch.classes.flashoverlap_class.OverlapImpl: the public class of the
// library.  Method names and argument lists follow the reference
// (reference: src/overlap_impl.h:9-40, src/pybind.cpp:129-144); both the
// upstream CUDA names (nccl_* / cutlass_*) and the names of the MUSA checkout
// (mccl_* / mutlass_*) are registered.  The overlapped operations run as one
// fused sm_100a kernel (FusedEngine); the non-overlapped ones run the same
// GEMM kernel followed by an NCCL collective on the same stream.
#pragma once

#include <torch/custom_class.h>
#include <torch/torch.h>

#include <memory>

#include "../runtime/engine.h"
#include "checks.h"
#include "nccl_utils.h"

namespace fo {

class OverlapImpl : public torch::CustomClassHolder {
 public:
  OverlapImpl();
  ~OverlapImpl() override;

  // ---- reference API ------------------------------------------------------
  void NcclInit(int64_t rank, int64_t size, std::vector<int64_t> id);
  void CutlassInit();
  void OverlapInit();
  void Gemm(at::Tensor A, at::Tensor B, at::Tensor C, int64_t algo);
  void GemmAllReduceOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor MM, at::Tensor RA, int64_t rLDN,
                            at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t algo, bool if_monitor);
  // (C is scratch: in the reference it holds this rank's partial products for
  // NCCL to read; the fused kernel stages partials in symmetric memory instead
  // and leaves C untouched.)
  void GemmReduceScatterOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor MM, at::Tensor RA,
                                at::Tensor RE, int64_t rLDN, at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t algo,
                                bool if_monitor);
  void GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C, int64_t algo);
  void GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t algo);
  void GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t algo, at::Tensor mLen_CPU);
  void NcclAllReduce(at::Tensor C);
  void NcclReduceScatter(at::Tensor C);
  void NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU);
  void SegAllReduce(at::Tensor C, at::Tensor cSEG_CPU, int64_t SegNum);

  // ---- the reference's own overlap design, restated for B200 ---------------
  // Comparator, not the product: a signalling GEMM on the current stream counts
  // finished tiles per segment in MM; a second, high-priority stream waits for
  // each segment's count with a stream memory operation (cuStreamWaitValue32:
  // no kernel spins, unlike the reference's kernel_wait_flag) and then runs
  // NCCL all-reduce / reduce-scatter on that segment of the tile-reordered
  // buffer (reference: src/overlap_impl.cu:221-328).  `gemm_ctas` CTAs compute
  // (0 = SM count - 16, leaving SMs to the NCCL kernels).  MM is left at zero.
  void GemmAllReduceTwoStream(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor MM, at::Tensor RA, int64_t rLDN,
                              at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t algo, int64_t gemm_ctas);
  void GemmReduceScatterTwoStream(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor MM,
                                  at::Tensor RA, at::Tensor RE, int64_t rLDN, at::Tensor cSEG_CPU,
                                  at::Tensor cSEG_GPU, int64_t algo, int64_t gemm_ctas);

  // ---- fused entry points with natural-order results ----------------------
  // GEMM + all-reduce (+ RMSNorm when `weight` is given).  Returns a tensor
  // that aliases the symmetric result buffer (valid until the second next
  // fused call on this object).
  at::Tensor GemmAllReduceFused(at::Tensor A, at::Tensor B, c10::optional<at::Tensor> weight, double eps,
                                int64_t algo);
  // GEMM + reduce-scatter (+ RMSNorm) into D [M/size, N].
  void GemmReduceScatterFused(at::Tensor A, at::Tensor B, at::Tensor D, c10::optional<at::Tensor> weight, double eps,
                              int64_t algo, bool interleave);
  // All-gather + GEMM in one launch: A_shard is this rank's [M/size, K] rows,
  // C receives gather(A)[M, K] * B[N, K]^T.
  void AllGatherGemm(at::Tensor A_shard, at::Tensor B, at::Tensor C, int64_t algo);
  // All-to-all dispatch + GEMM in one launch (see FusedEngine::a2a_gemm):
  // A_send holds the rows for rank 0, 1, ... back to back, mLen_CPU[i][j] rows
  // go from rank i to rank j, C needs a2a_padded_rows(mLen_CPU, algo) rows.
  void A2aDispatchGemm(at::Tensor A_send, at::Tensor B, at::Tensor C, at::Tensor mLen_CPU, int64_t algo);
  int64_t A2aPaddedRows(at::Tensor mLen_CPU, int64_t algo);
  // GEMM + RMSNorm on one GPU: C receives A*B^T, O the normalised rows.
  void GemmRmsNorm(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor O, at::Tensor weight, double eps,
                   int64_t algo);

  // Collective.  Gives the object symmetric memory allocated elsewhere:
  // `peer_ptrs[r]` is rank r's buffer mapped into this process, `mc_ptr` the
  // multicast address (0 = none), `nbytes` the size of each buffer.  With a
  // multicast address the fused operations reduce through NVLink SHARP.
  void AttachSymmetric(std::vector<int64_t> peer_ptrs, int64_t mc_ptr, int64_t nbytes);
  // Collective.  Drops the attached memory again (used when some rank could not map it).
  void DetachSymmetric();
  void SetUseNvls(bool allreduce, bool reducescatter);
  // All-gather -> GEMM: true pushes the shard through the switch (one multimem.st
  // per chunk, needs a multicast mapping); false (default) = ring of peer-to-peer stores.
  void SetAllGatherMulticast(bool on);
  bool NvlsAvailable();
  // Whether the fused all-reduce currently takes the NVLink SHARP path.
  bool AllReduceUsesNvls();

  // Collective: all-to-all push of `bytes` per peer with the P2P store kernel
  // (bandwidth tool); `ctas` = 0 uses every SM.
  void P2pPush(int64_t bytes, int64_t ctas);
  // Same with bulk copies from shared memory, `chunk_bytes` per copy.
  void P2pPushBulk(int64_t bytes, int64_t chunk_bytes, int64_t ctas);
  // Collective NVLink SHARP primitive over `bytes` of symmetric memory:
  // kind "ld_reduce" | "st" | "allreduce"; each rank handles its 1/size share.
  void MultimemBench(std::string kind, int64_t bytes, int64_t ctas, bool bf16);

  // ---- transport ---------------------------------------------------------
  // "p2p" (default on one node): the fused kernels move data through
  // peer-mapped memory.  "nccl": ranks that cannot map each other's memory
  // (several nodes) keep every entry point working on NCCL: the overlap calls
  // run the two-stream design, the fused calls run GEMM, one NCCL collective and
  // the RMSNorm kernel.  nccl_init selects "nccl" by itself when the ranks sit
  // on different hosts.
  void SetTransport(std::string name);
  std::string Transport();

  // ---- tuning knobs and failure reporting ---------------------------------
  // Failure-path self test, see FusedEngine::wait_on_unset_counter.
  void WaitOnUnsetCounter(int64_t timeout_ms);
  void SetTimeoutMs(int64_t ms);
  void SetSmCount(int64_t n);
  void SetRasterGroup(int64_t g);
  // L2 eviction hints on the GEMM's operand loads (default off).
  void SetL2Hints(bool on);
  // Shrinking last raster groups in operations with a reduce phase (default on).
  void SetRasterTaper(bool on);
  // Every following launch records per-CTA phase timestamps into `buf`
  // (int64, at least 8 * SM count entries, layout in FusedParams::phase_trace;
  // an empty tensor turns it off).
  void SetPhaseTrace(at::Tensor buf);
  // Every following fused launch whose M is at most rows records a timeline of
  // its reduce phase into `buf` (int64 [6, rows]: claimed, stored, CTA * 4 +
  // row group, partials there, summed, barrier passed; times as %globaltimer ns; an empty tensor turns it off).
  void SetRowTrace(at::Tensor buf);
  // [code, rank, where, seen, want]; code 0 = no failure reported.
  std::vector<int64_t> Status();
  std::string StatusString();
  // Raises if a kernel reported a failure.
  void CheckStatus();
  void Reset();
  int64_t NumAlgos();
  std::vector<int64_t> AlgoTile(int64_t algo);

 private:
  GemmOperands operands(const at::Tensor& A, const at::Tensor& B, int64_t algo) const;
  void require_comm(const char* op) const;

  void two_stream(bool scatter, at::Tensor& A, at::Tensor& B, at::Tensor& C, at::Tensor* D, at::Tensor& MM,
                  at::Tensor& RA, at::Tensor* RE, int64_t rLDN, at::Tensor& cSEG_CPU, at::Tensor& cSEG_GPU,
                  int64_t algo, int64_t gemm_ctas, bool monitor);
  Communicator comm_;
  FusedEngine engine_;
  cudaStream_t comm_stream_ = nullptr;
  cudaEvent_t join_event_ = nullptr;
  cudaEvent_t raise_event_ = nullptr;
  IndexCheckCache index_checks_;  // RA / RE tensors already validated
  bool nccl_transport_ = false;
  bool engine_ready_ = false;
  at::Tensor phase_trace_;
  at::Tensor row_trace_;
};

}  // namespace fo
