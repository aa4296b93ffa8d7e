#include "engine.h"

#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <cstring>
#include <sstream>
#include <stdexcept>

namespace fo {

namespace {
// NVTX range around every public operation (visible in Nsight Systems; a few
// nanoseconds when no tool is attached).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(cuda_error_string(e, what));
}
void check_launch(cudaError_t e, const char* why, const char* op) {
  if (e != cudaSuccess) {
    std::string msg = std::string(op) + ": " + (why && *why ? why : "launch failed");
    throw std::runtime_error(cuda_error_string(e, msg.c_str()));
  }
}
}  // namespace

FusedEngine::~FusedEngine() {
  if (status_dev_ != nullptr) cudaFree(status_dev_);
  if (status_host_ != nullptr) cudaFreeHost(status_host_);
  status_dev_ = nullptr;
  status_host_ = status_mirror_ = nullptr;
}

void FusedEngine::init(int rank, int world, AllGatherFn all_gather) {
  if (world < 1 || world > kMaxRanks) throw std::runtime_error("FusedEngine: world size must be 1..8");
  if (rank < 0 || rank >= world) throw std::runtime_error("FusedEngine: bad rank");
  rank_ = rank;
  world_ = world;
  all_gather_ = std::move(all_gather);
  if (status_dev_ == nullptr) {
    check(cudaMalloc(reinterpret_cast<void**>(&status_dev_), sizeof(StatusWord)), "cudaMalloc(status)");
    check(cudaMemset(status_dev_, 0, sizeof(StatusWord)), "cudaMemset(status)");
    // mirror in mapped host memory: read by check_previous() without a synchronisation
    check(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), sizeof(StatusWord), cudaHostAllocMapped),
          "cudaHostAlloc(status mirror)");
    std::memset(status_host_, 0, sizeof(StatusWord));
    check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_mirror_), status_host_, 0),
          "cudaHostGetDevicePointer(status mirror)");
  }
}

void FusedEngine::check_previous(const char* op) const {
  if (status_host_ == nullptr) return;
  const volatile StatusWord* m = status_host_;
  if (m->code == ST_OK) return;
  StatusWord s;
  s.code = m->code;
  s.rank = m->rank;
  s.where = m->where;
  s.seen = m->seen;
  s.want = m->want;
  throw std::runtime_error(std::string(op) + ": an earlier flashoverlap kernel reported a failure: " + describe(s) +
                           "; its results are not valid (reset() clears the state)");
}

uint32_t* FusedEngine::flag_ptr(int rank, int set) const {
  return static_cast<uint32_t*>(heap_.ptr(rank, ws_.flags[set]));
}
uint32_t* FusedEngine::done_ptr(int rank, int set) const { return flag_ptr(rank, set) + kFlagDone; }

namespace {
size_t workspace_bytes(long long elems) {
  const size_t mat = static_cast<size_t>(elems) * 2;
  return 4 * (mat + 4096) + 3 * (kFlagWords * 4 + 4096) + 8192 + (1 << 20);
}
}  // namespace

void FusedEngine::carve_workspace(long long elems) {
  const size_t mat = static_cast<size_t>(elems) * 2;
  heap_.reset_allocator();
  for (int s = 0; s < 2; ++s) ws_.stage[s] = heap_.alloc(mat, 1024);
  for (int s = 0; s < 2; ++s) ws_.result[s] = heap_.alloc(mat, 1024);
  for (int s = 0; s < 2; ++s) ws_.flags[s] = heap_.alloc(kFlagWords * 4, 1024);
  ws_.misc = heap_.alloc(4096, 1024);
  ws_.local_flags = heap_.alloc(kFlagWords * 4, 1024);
  ws_.capacity_elems = elems;
  calls_ = 0;
  pushes_ = 0;
  mm_arrivals_ = 0;
}

void FusedEngine::attach_symmetric(size_t bytes, const std::vector<void*>& peer_ptrs, void* mc_ptr) {
  if (!initialized()) throw std::runtime_error("attach_symmetric: engine not initialised");
  if (heap_.valid()) {
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    heap_.destroy();
  }
  heap_.attach(rank_, world_, bytes, peer_ptrs, mc_ptr);
  check(cudaMemset(heap_.local(0), 0, bytes), "cudaMemset(symmetric memory)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (world_ > 1 && all_gather_) {  // nobody signals into memory that is not zeroed yet
    char t = 1;
    std::vector<char> all(world_);
    all_gather_(&t, 1, all.data());
  }
  // the largest problem the attached memory can hold
  long long elems = static_cast<long long>((bytes - workspace_bytes(0)) / 8);
  if (elems < 1) throw std::runtime_error("attach_symmetric: buffer too small");
  carve_workspace(elems);
}

void FusedEngine::detach_symmetric() {
  if (!heap_.valid() || heap_.owned()) return;
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  heap_.destroy();
  ws_ = Workspace{};
  calls_ = 0;
  pushes_ = 0;
  mm_arrivals_ = 0;
}

void FusedEngine::ensure_workspace(long long m, long long n) {
  const long long elems = m * n;
  if (heap_.valid() && ws_.capacity_elems >= elems) return;
  if (heap_.valid() && !heap_.owned()) {
    throw std::runtime_error("the attached symmetric memory is too small for this problem: need " +
                             std::to_string(workspace_bytes(elems)) + " bytes");
  }
  if (heap_.valid()) {
    // Growing: all ranks get here in the same call.  Drain the device, then a
    // gather as a barrier so that no peer still writes into the old slab.
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (world_ > 1) {
      char t = 1;
      std::vector<char> all(world_);
      all_gather_(&t, 1, all.data());
    }
    heap_.destroy();
  }
  heap_.init(rank_, world_, workspace_bytes(elems), all_gather_);
  carve_workspace(elems);
}

void FusedEngine::base_params(FusedParams& p, const SignalArgs* sig) {
  p = FusedParams{};
  if (sig != nullptr) {
    p.seg_counter = sig->seg_counter;
    p.cseg = sig->cseg;
    p.nseg = sig->nseg;
    p.ticket_counter = sig->ticket_counter;
    p.trace = sig->trace;
    p.slot_of_tile = sig->slot_of_tile;
  }
  p.ws = world_;
  p.me = rank_;
  p.status = status_dev_;
  p.status_mirror = status_mirror_;
  p.timeout_ns = timeout_ns_;
  p.raster_group = raster_group_;
  p.l2_hints = l2_hints_ ? 1 : 0;
  p.raster_taper = 0;  // set by the operations that have a reduce phase
  p.phase_trace = phase_trace_;
  p.row_trace = nullptr;  // set by the operations with a reduce phase when the buffer is large enough
  p.epi_layout.ld = 0;
}

void FusedEngine::gemm(const GemmOperands& g_in, void* C, const OutLayout* layout, const SignalArgs* sig,
                       cudaStream_t stream) {
  NvtxRange range("flashoverlap::gemm");
  if (!initialized()) init(0, 1, nullptr);
  check_previous("gemm");
  FusedParams p;
  base_params(p, sig);
  GemmOperands g = g_in;
  if (g.sm_count == 0) g.sm_count = sm_count_;
  p.own_mode = OWN_SINGLE;
  p.ws = 1;
  p.me = 0;
  p.rows_per_owner = g.M;
  p.epi_base[0] = C;
  if (layout != nullptr) p.epi_layout = *layout;
  else p.epi_layout.ld = g.N;
  if (p.raster_group == 0) p.raster_group = 8;
  const char* why = nullptr;
  check_launch(launch_fused(g, p, stream, &why), why, "gemm");
}

void FusedEngine::gemm_rmsnorm(const GemmOperands& g_in, void* scratch, void* out, const NormArgs& norm,
                               cudaStream_t stream) {
  NvtxRange range("flashoverlap::gemm_rmsnorm");
  if (!initialized()) init(0, 1, nullptr);
  check_previous("gemm_rmsnorm");
  ensure_workspace(1, 1);  // only the counters are needed
  GemmOperands g = g_in;
  if (g.sm_count == 0) g.sm_count = sm_count_;
  const TileConfig tc = algo_config(g.algo);
  if (g.M / 128 > kMaxTileRows) throw std::runtime_error("gemm_rmsnorm: too many tile rows");
  // A purely local operation: it uses its own counters, cleared right before the
  // launch, and does not take part in the alternation of the shared sets (it
  // does not synchronise the ranks, so it must not advance their call count).
  uint32_t* local = static_cast<uint32_t*>(heap_.local(ws_.local_flags));
  check(cudaMemsetAsync(local, 0, kFlagWords * 4, stream), "cudaMemsetAsync(counters)");
  FusedParams p;
  base_params(p, nullptr);
  p.own_mode = OWN_SINGLE;
  p.ws = 1;
  p.me = 0;
  p.rows_per_owner = g.M;
  p.epi_base[0] = scratch;
  p.epi_layout.ld = g.N;
  p.flag[0] = local;
  p.job_counter = local + kFlagJob;
  if (p.raster_group == 0) p.raster_group = 8;
  p.raster_taper = raster_taper_ ? 1 : 0;
  p.reduce = 1;
  if (row_trace_ != nullptr && g.M <= row_trace_rows_) p.row_trace = row_trace_;
  p.stage = scratch;
  p.flag_target = static_cast<uint32_t>(g.N / tc.bn);
  p.norm = norm.gamma != nullptr;
  p.gamma = norm.gamma;
  p.eps = norm.eps;
  p.bcast = 0;
  p.out[0] = out;
  p.out_layout.ld = g.N;
  const char* why = nullptr;
  check_launch(launch_fused(g, p, stream, &why), why, "gemm_rmsnorm");
}

void* FusedEngine::gemm_allreduce(const GemmOperands& g_in, void* out_user, const NormArgs& norm,
                                  const OutLayout* out_layout, const SignalArgs* sig, cudaStream_t stream) {
  NvtxRange range("flashoverlap::gemm_allreduce");
  if (!initialized()) throw std::runtime_error("gemm_allreduce: engine not initialised");
  check_previous("gemm_allreduce");
  GemmOperands g = g_in;
  if (g.sm_count == 0) g.sm_count = sm_count_;
  const TileConfig tc = algo_config(g.algo);
  if (g.M % world_ != 0) throw std::runtime_error("gemm_allreduce: M must be divisible by the world size");
  if (g.M / 128 > kMaxTileRows) throw std::runtime_error("gemm_allreduce: too many tile rows");
  ensure_workspace(g.M, g.N);
  const int set = static_cast<int>(calls_ & 1ull);
  check(cudaMemsetAsync(flag_ptr(rank_, set ^ 1), 0, kFlagWords * 4, stream), "cudaMemsetAsync(counters)");
  if (world_ == 1 && norm.gamma == nullptr && sig == nullptr && out_layout == nullptr) {
    // One rank and no RMSNorm: nothing to sum or scale, the GEMM writes the result itself.  The buffer
    // sets still alternate (and the other set's counters are cleared above) like after any fused call.
    void* result = out_user != nullptr ? out_user : heap_.local(ws_.result[set]);
    gemm(g, result, nullptr, nullptr, stream);
    ++calls_;
    return result;
  }

  FusedParams p;
  base_params(p, sig);
  const int rows_local = g.M / world_;
  p.own_mode = world_ == 1 ? OWN_SINGLE : OWN_INTERLEAVE;
  p.rows_per_owner = rows_local;
  const size_t slot_bytes = static_cast<size_t>(rows_local) * g.N * 2;
  for (int r = 0; r < world_; ++r) {
    // my slot inside owner r's staging buffer
    p.epi_base[r] = static_cast<char*>(heap_.ptr(r, ws_.stage[set])) + slot_bytes * rank_;
    p.flag[r] = flag_ptr(r, set);
    p.out[r] = heap_.ptr(r, ws_.result[set]);
    p.done[r] = done_ptr(r, set);
  }
  p.epi_layout.ld = g.N;
  if (allreduce_uses_nvls()) {
    p.nvls = 1;
    p.epi_base[0] = heap_.local(ws_.stage[set]);  // partials stay here, [M][N]
    p.mc_stage = heap_.mc(ws_.stage[set]);
    p.mc_flag = static_cast<uint32_t*>(heap_.mc(ws_.flags[set]));
    p.mc_out = heap_.mc(ws_.result[set]);
    p.mc_done = static_cast<uint32_t*>(heap_.mc(ws_.flags[set])) + kFlagDone;
  }
  // one GPU: wide groups for L2 reuse; several GPUs: narrow groups so that tile rows complete early
  if (p.raster_group == 0) p.raster_group = world_ == 1 ? 8 : 2;
  p.raster_taper = raster_taper_ ? 1 : 0;
  p.reduce = 1;
  if (row_trace_ != nullptr && g.M <= row_trace_rows_) p.row_trace = row_trace_;
  p.stage = heap_.local(ws_.stage[set]);
  p.flag_target = static_cast<uint32_t>(world_ * (g.N / tc.bn));
  p.norm = norm.gamma != nullptr;
  p.gamma = norm.gamma;
  p.eps = norm.eps;
  // with one rank there is nobody to deliver to: rows go to the result buffer like a reduce-scatter's
  p.bcast = world_ > 1 ? 1 : 0;
  if (out_layout != nullptr) p.out_layout = *out_layout;
  else p.out_layout.ld = g.N;
  p.done_target = static_cast<uint32_t>(g.M) * kGroupWarps;  // one delivery count per warp and row
  p.job_counter = flag_ptr(rank_, set) + kFlagJob;
  const char* why = nullptr;
  check_launch(launch_fused(g, p, stream, &why), why, "gemm_allreduce");
  ++calls_;
  void* result = heap_.local(ws_.result[set]);
  if (out_user != nullptr) {
    check(cudaMemcpyAsync(out_user, result, static_cast<size_t>(g.M) * g.N * 2, cudaMemcpyDeviceToDevice, stream),
          "cudaMemcpyAsync(result)");
  }
  return result;
}

void FusedEngine::gemm_reducescatter(const GemmOperands& g_in, void* D, bool interleave, const NormArgs& norm,
                                     const OutLayout* out_layout, const SignalArgs* sig, cudaStream_t stream) {
  NvtxRange range("flashoverlap::gemm_reducescatter");
  if (!initialized()) throw std::runtime_error("gemm_reducescatter: engine not initialised");
  check_previous("gemm_reducescatter");
  GemmOperands g = g_in;
  if (g.sm_count == 0) g.sm_count = sm_count_;
  const TileConfig tc = algo_config(g.algo);
  if (g.M % world_ != 0) throw std::runtime_error("gemm_reducescatter: M must be divisible by the world size");
  if (g.M / 128 > kMaxTileRows) throw std::runtime_error("gemm_reducescatter: too many tile rows");
  const int rows_local = g.M / world_;
  if (!interleave && world_ > 1 && rows_local % tc.bm != 0) {
    throw std::runtime_error("gemm_reducescatter: contiguous ownership needs (M / world) to be a multiple of the tile "
                             "height (" + std::to_string(tc.bm) + " for this Algo)");
  }
  ensure_workspace(g.M, g.N);
  const int set = static_cast<int>(calls_ & 1ull);
  check(cudaMemsetAsync(flag_ptr(rank_, set ^ 1), 0, kFlagWords * 4, stream), "cudaMemsetAsync(counters)");
  if (world_ == 1 && norm.gamma == nullptr && sig == nullptr && out_layout == nullptr) {
    gemm(g, D, nullptr, nullptr, stream);  // one rank, no RMSNorm: the GEMM writes the rows where they belong
    ++calls_;
    return;
  }

  FusedParams p;
  base_params(p, sig);
  p.own_mode = world_ == 1 ? OWN_SINGLE : (interleave ? OWN_INTERLEAVE : OWN_BLOCK);
  p.rows_per_owner = rows_local;
  const size_t slot_bytes = static_cast<size_t>(rows_local) * g.N * 2;
  for (int r = 0; r < world_; ++r) {
    p.epi_base[r] = static_cast<char*>(heap_.ptr(r, ws_.stage[set])) + slot_bytes * rank_;
    p.flag[r] = flag_ptr(r, set);
  }
  p.epi_layout.ld = g.N;
  if (reducescatter_uses_nvls()) {
    p.nvls = 1;
    p.epi_base[0] = heap_.local(ws_.stage[set]);
    p.mc_stage = heap_.mc(ws_.stage[set]);
    p.mc_flag = static_cast<uint32_t*>(heap_.mc(ws_.flags[set]));
  }
  if (p.own_mode == OWN_BLOCK) {
    // the walk cycles through the owners (a different first owner on every rank): all links are busy at
    // any moment and every owner's rows complete progressively instead of all at the end
    p.owner_stride = rows_local / tc.bm;
  }
  // one GPU: wide groups for L2 reuse; several GPUs: narrow groups so that tile rows complete early
  if (p.raster_group == 0) {
    // several ranks: a quarter of the tile rows per group, between 2 and 8 (timed on 2 and 4 GPUs: rows
    // must start completing early, but small groups stream all of B once per group)
    int rg = (g.M / tc.bm) / 4;
    rg = rg < 2 ? 2 : (rg > 8 ? 8 : rg);
    p.raster_group = world_ == 1 ? 8 : rg;
  }
  p.raster_taper = raster_taper_ ? 1 : 0;
  p.reduce = 1;
  if (row_trace_ != nullptr && g.M <= row_trace_rows_) p.row_trace = row_trace_;
  p.stage = heap_.local(ws_.stage[set]);
  p.flag_target = static_cast<uint32_t>(world_ * (g.N / tc.bn));
  p.norm = norm.gamma != nullptr;
  p.gamma = norm.gamma;
  p.eps = norm.eps;
  p.bcast = 0;
  p.job_counter = flag_ptr(rank_, set) + kFlagJob;
  p.out[rank_] = D;
  if (out_layout != nullptr) p.out_layout = *out_layout;
  else p.out_layout.ld = g.N;
  const char* why = nullptr;
  check_launch(launch_fused(g, p, stream, &why), why, "gemm_reducescatter");
  ++calls_;
}

// Common part of all-gather -> GEMM and all-to-all dispatch -> GEMM.
// src_for[r] / bytes_for[r]: what this rank sends to rank r; src_end[r]: end row
// of source r's block in this rank's gathered buffer; M: rows of the
// gathered buffer that take part in the GEMM (multiple of the tile height);
// first_row: where this rank's own block starts (the GEMM begins there).
void FusedEngine::gathered_gemm(const void* const* src_for, const long long* bytes_for, const int* src_end, int M,
                                int first_row, const void* B, void* C, int N, int K, DType dtype, int algo,
                                const char* op, cudaStream_t stream, size_t mc_slot_offset, const void* a_own,
                                int own_rows) {
  NvtxRange range(op);
  const TileConfig tc = algo_config(algo);
  const int set = static_cast<int>(calls_ & 1ull);
  check(cudaMemsetAsync(flag_ptr(rank_, set ^ 1), 0, kFlagWords * 4, stream), "cudaMemsetAsync(counters)");
  FusedParams p;
  base_params(p, nullptr);
  GemmOperands g{};
  g.A = heap_.local(ws_.stage[set]);  // the gathered A of this call
  g.B = B;
  g.M = M;
  g.N = N;
  g.K = K;
  g.dtype = dtype;
  g.algo = algo;
  g.A_own = a_own;  // this rank's rows are read in place (all-gather), not from the gathered buffer
  g.own_begin = first_row;
  g.own_rows = a_own != nullptr ? own_rows : 0;
  p.own_mode = OWN_SINGLE;
  p.ws = world_;
  p.me = rank_;
  p.rows_per_owner = M;
  p.epi_base[0] = C;
  p.epi_layout.ld = N;
  if (p.raster_group == 0) p.raster_group = 2;
  p.rot = first_row / tc.bm;  // own rows first, then the blocks in the order they are pushed to this rank
  p.a_ready = flag_ptr(rank_, set) + kFlagAReady;
  p.ag_push = 1;
  for (int r = 0; r < world_; ++r) {
    p.a_src_end[r] = src_end[r];
    p.ag_src[r] = src_for[r];
    p.ag_bytes[r] = bytes_for[r];
    p.ag_flag[r] = flag_ptr(r, set) + kFlagAReady + rank_;
  }
  // every communication warp of every CTA pushes a share and bumps the counter once per destination
  int grid = sm_count_ > 0 ? sm_count_ : device_sm_count();
  if (grid > device_sm_count()) grid = device_sm_count();
  if (tc.ctas == 2) grid &= ~1;
  g.sm_count = grid;
  p.a_ready_target = static_cast<uint32_t>(grid) * kCommWarps;
  p.reduce = 0;
  p.force_full_grid = 1;
  // ag_dst is filled by the callers' layout: where my block lives on rank r
  for (int r = 0; r < world_; ++r) p.ag_dst[r] = ag_dst_scratch_[r];
  if (mc_slot_offset != kNoMulticast && nvls_available() && nvls_ag_) {
    // every rank receives the same rows: push them once through the switch
    p.ag_mc_dst = static_cast<char*>(heap_.mc(ws_.stage[set])) + mc_slot_offset;
    p.ag_mc_flag = static_cast<uint32_t*>(heap_.mc(ws_.flags[set])) + kFlagAReady + rank_;
  }
  const char* why = nullptr;
  check_launch(launch_fused(g, p, stream, &why), why, op);
  ++calls_;
}

void FusedEngine::allgather_gemm(const void* A_shard, const void* B, void* C, int M, int N, int K, DType dtype,
                                 int algo, cudaStream_t stream) {
  if (!initialized()) throw std::runtime_error("allgather_gemm: engine not initialised");
  check_previous("allgather_gemm");
  if (M % world_ != 0) throw std::runtime_error("allgather_gemm: M must be divisible by the world size");
  const int rows = M / world_;
  if (rows % 128 != 0) throw std::runtime_error("allgather_gemm: M / world must be a multiple of 128");
  if (K % 8 != 0) throw std::runtime_error("allgather_gemm: K must be a multiple of 8");
  if (world_ == 1 && reinterpret_cast<uintptr_t>(A_shard) % 16 == 0) {  // nothing to gather: the GEMM reads the caller's matrix
    GemmOperands g{};
    g.A = A_shard;
    g.B = B;
    g.M = M;
    g.N = N;
    g.K = K;
    g.dtype = dtype;
    g.algo = algo;
    gemm(g, C, nullptr, nullptr, stream);
    return;
  }
  ensure_workspace(static_cast<long long>(M) * (K > N ? K : N), 1);
  const int set = static_cast<int>(calls_ & 1ull);
  const size_t shard_bytes = static_cast<size_t>(rows) * K * 2;
  const void* src_for[kMaxRanks];
  long long bytes_for[kMaxRanks];
  int src_end[kMaxRanks];
  // The GEMM reads this rank's own rows straight from the caller's shard (a second TMA descriptor), so
  // they are not copied into the gathered buffer: nothing is sent to `rank_` itself (the counter is
  // still bumped).  With the multicast push every rank, this one included, receives the copy anyway.
  const bool in_place = reinterpret_cast<uintptr_t>(A_shard) % 16 == 0;
  const bool multicast_push = nvls_available() && nvls_ag_;  // takes the shard's size from the entry of this rank
  for (int r = 0; r < world_; ++r) {
    src_for[r] = A_shard;
    bytes_for[r] = (r == rank_ && in_place && !multicast_push) ? 0 : static_cast<long long>(shard_bytes);
    src_end[r] = (r + 1) * rows;
    ag_dst_scratch_[r] = static_cast<char*>(heap_.ptr(r, ws_.stage[set])) + shard_bytes * rank_;
  }
  gathered_gemm(src_for, bytes_for, src_end, M, rank_ * rows, B, C, N, K, dtype, algo, "allgather_gemm", stream,
                shard_bytes * rank_, in_place ? A_shard : nullptr, rows);
}

int FusedEngine::a2a_padded_rows(const int* mlen, int algo) const {
  const TileConfig tc = algo_config(algo);
  int most = 0;
  for (int j = 0; j < world_; ++j) {
    int recv = 0;
    for (int i = 0; i < world_; ++i) recv += mlen[i * world_ + j];
    if (recv > most) most = recv;
  }
  if (most == 0) most = 1;
  return (most + tc.bm - 1) / tc.bm * tc.bm;
}

void FusedEngine::a2a_gemm(const void* A_send, const void* B, void* C, const int* mlen, int N, int K, DType dtype,
                           int algo, cudaStream_t stream) {
  if (!initialized()) throw std::runtime_error("a2a_gemm: engine not initialised");
  check_previous("a2a_gemm");
  if (K % 8 != 0) throw std::runtime_error("a2a_gemm: K must be a multiple of 8");
  for (int i = 0; i < world_ * world_; ++i) {
    if (mlen[i] < 0) throw std::runtime_error("a2a_gemm: negative row count");
  }
  const int m_pad = a2a_padded_rows(mlen, algo);  // the same on every rank
  if (world_ == 1 && mlen[0] == m_pad && reinterpret_cast<uintptr_t>(A_send) % 16 == 0) {  // one rank, whole tiles: in place
    GemmOperands g{};
    g.A = A_send;
    g.B = B;
    g.M = m_pad;
    g.N = N;
    g.K = K;
    g.dtype = dtype;
    g.algo = algo;
    gemm(g, C, nullptr, nullptr, stream);
    return;
  }
  ensure_workspace(static_cast<long long>(m_pad) * (K > N ? K : N), 1);
  const int set = static_cast<int>(calls_ & 1ull);
  const size_t row_bytes = static_cast<size_t>(K) * 2;
  const void* src_for[kMaxRanks];
  long long bytes_for[kMaxRanks];
  int src_end[kMaxRanks];
  size_t send_off = 0;
  int first_row = 0;
  for (int r = 0; r < world_; ++r) {
    // what I send to r, and where it lands there: behind the rows of the sources before me
    src_for[r] = static_cast<const char*>(A_send) + send_off;
    bytes_for[r] = static_cast<long long>(mlen[rank_ * world_ + r]) * static_cast<long long>(row_bytes);
    send_off += static_cast<size_t>(bytes_for[r]);
    size_t before = 0;
    for (int i = 0; i < rank_; ++i) before += static_cast<size_t>(mlen[i * world_ + r]);
    ag_dst_scratch_[r] = static_cast<char*>(heap_.ptr(r, ws_.stage[set])) + before * row_bytes;
  }
  int acc = 0;
  for (int i = 0; i < world_; ++i) {
    if (i == rank_) first_row = acc;
    acc += mlen[i * world_ + rank_];
    src_end[i] = acc;
  }
  // This rank multiplies the rows it received, rounded up to whole tiles (rows
  // between `acc` and that height belong to nobody: the GEMM reads whatever an
  // earlier call left there and writes scratch rows of C).  Ranks that received
  // fewer rows launch a smaller GEMM; the workspace is sized for the largest.
  const TileConfig tc_own = algo_config(algo);
  int m_own = (acc + tc_own.bm - 1) / tc_own.bm * tc_own.bm;
  if (m_own < tc_own.bm) m_own = tc_own.bm;
  if (m_own > m_pad) m_own = m_pad;
  gathered_gemm(src_for, bytes_for, src_end, m_own, first_row, B, C, N, K, dtype, algo, "a2a_gemm", stream,
                kNoMulticast, nullptr, 0);  // every destination gets different rows; own rows are copied (ragged blocks)
}

void FusedEngine::p2p_push(long long bytes, int ctas, cudaStream_t stream) {
  NvtxRange range("flashoverlap::p2p_push");
  push_common(bytes, 0, ctas, stream);
}

void FusedEngine::p2p_push_bulk(long long bytes, int chunk_bytes, int ctas, cudaStream_t stream) {
  NvtxRange range("flashoverlap::p2p_push_bulk");
  if (chunk_bytes < 16 || chunk_bytes > 16384 || chunk_bytes % 16 != 0) {
    throw std::runtime_error("p2p_push_bulk: chunk_bytes must be a multiple of 16 in [16, 16384]");
  }
  push_common(bytes, chunk_bytes, ctas, stream);
}

void FusedEngine::push_common(long long bytes, int chunk_bytes, int ctas, cudaStream_t stream) {
  if (!initialized()) throw std::runtime_error("p2p_push: engine not initialised");
  check_previous("p2p_push");
  if (bytes <= 0 || bytes % 16 != 0) throw std::runtime_error("p2p_push: bytes must be a positive multiple of 16");
  ensure_workspace(static_cast<long long>(world_) * bytes / 2 + 8, 1);
  if (ctas <= 0) ctas = device_sm_count();
  PushParams p{};
  p.src = heap_.local(ws_.stage[0]);
  p.bytes = bytes;
  p.src_stride = 0;
  p.ws = world_;
  p.me = rank_;
  p.include_self = 0;
  for (int r = 0; r < world_; ++r) {
    p.dst[r] = static_cast<char*>(heap_.ptr(r, ws_.result[0])) + static_cast<size_t>(rank_) * bytes;
    p.flag[r] = static_cast<uint32_t*>(heap_.ptr(r, ws_.misc));
  }
  if (chunk_bytes > 0) check(launch_p2p_push_bulk(p, chunk_bytes, ctas, stream), "p2p_push_bulk launch");
  else check(launch_p2p_push(p, ctas, stream), "p2p_push launch");
  pushes_ += static_cast<unsigned long long>(world_ - 1) * ctas;  // arrivals expected here so far
  if (world_ > 1) {
    const uint32_t target = static_cast<uint32_t>(pushes_);
    check(launch_wait_counter(static_cast<uint32_t*>(heap_.local(ws_.misc)), target, timeout_ns_, status_dev_, status_mirror_, rank_,
                              stream),
          "wait_counter launch");
  }
}

void FusedEngine::multimem_bench(int kind, long long bytes, int ctas, DType dtype, cudaStream_t stream) {
  NvtxRange range("flashoverlap::multimem_bench");
  if (!initialized()) throw std::runtime_error("multimem_bench: engine not initialised");
  check_previous("multimem_bench");
  if (kind < MM_LD_REDUCE || kind > MM_ALLREDUCE) throw std::runtime_error("multimem_bench: unknown kind");
  if (bytes <= 0 || bytes % (16 * world_) != 0) {
    throw std::runtime_error("multimem_bench: bytes must be a positive multiple of 16 * world");
  }
  ensure_workspace(bytes / 2, 1);
  if (!nvls_available()) throw std::runtime_error("multimem_bench: the symmetric memory has no multicast mapping");
  if (ctas <= 0) ctas = device_sm_count();
  MultimemParams p{};
  p.kind = kind;
  p.bf16 = dtype == DT_BF16;
  p.mc_stage = heap_.mc(ws_.stage[0]);
  p.mc_result = heap_.mc(ws_.result[0]);
  p.local_src = heap_.local(ws_.stage[1]);
  p.local_dst = heap_.local(ws_.result[1]);
  p.bytes = bytes / world_;
  p.offset = p.bytes * rank_;
  p.mc_arrive = static_cast<uint32_t*>(heap_.mc(ws_.misc)) + 1;
  check(launch_multimem(p, ctas, stream), "multimem launch");
  mm_arrivals_ += static_cast<unsigned long long>(world_) * ctas;
  check(launch_wait_counter(static_cast<uint32_t*>(heap_.local(ws_.misc)) + 1, static_cast<uint32_t>(mm_arrivals_),
                            timeout_ns_, status_dev_, status_mirror_, rank_, stream),
        "wait_counter launch");
}

void FusedEngine::wait_on_unset_counter(long long timeout_ms, cudaStream_t stream) {
  if (!initialized()) init(0, 1, nullptr);
  if (world_ == 1) ensure_workspace(1, 1);
  if (!heap_.valid()) throw std::runtime_error("wait_on_unset_counter: no workspace yet");
  // word 512 of the private counter page is never written by any kernel
  const uint32_t* never = static_cast<uint32_t*>(heap_.local(ws_.misc)) + 512;
  check(launch_wait_counter(never, 1u, static_cast<unsigned long long>(timeout_ms) * 1000000ull, status_dev_,
                            status_mirror_, rank_,
                            stream),
        "wait_counter launch");
}

StatusWord FusedEngine::read_status() {
  StatusWord s{};
  if (status_dev_ == nullptr) return s;
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  check(cudaMemcpy(&s, status_dev_, sizeof(s), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
  return s;
}

void FusedEngine::clear_status() {
  if (status_dev_ != nullptr) check(cudaMemset(status_dev_, 0, sizeof(StatusWord)), "cudaMemset(status)");
  if (status_host_ != nullptr) std::memset(status_host_, 0, sizeof(StatusWord));
}

void FusedEngine::reset_counters() {
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (world_ > 1 && all_gather_) {
    char t = 1;
    std::vector<char> all(world_);
    all_gather_(&t, 1, all.data());
  }
  if (heap_.valid()) {
    for (int s = 0; s < 2; ++s) check(cudaMemset(flag_ptr(rank_, s), 0, kFlagWords * 4), "cudaMemset(counters)");
    check(cudaMemset(heap_.local(ws_.misc), 0, 4096), "cudaMemset(counters)");
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  }
  if (world_ > 1 && all_gather_) {
    char t = 1;
    std::vector<char> all(world_);
    all_gather_(&t, 1, all.data());
  }
  calls_ = 0;
  pushes_ = 0;
  mm_arrivals_ = 0;
  clear_status();
}

std::string FusedEngine::describe(const StatusWord& s) {
  static const char* names[] = {"ok",
                                "a pipeline barrier inside the GEMM timed out",
                                "partial results from a rank did not arrive in time",
                                "all-reduce results from an owner did not arrive in time",
                                "an index array held an out-of-range entry",
                                "an all-gathered operand shard did not arrive in time"};
  std::ostringstream os;
  os << (s.code < 6 ? names[s.code] : "unknown") << " [code " << s.code << ", rank " << s.rank << ", where 0x"
     << std::hex << s.where << std::dec << ", saw " << s.seen << ", wanted " << s.want << "]";
  return os.str();
}

}  // namespace fo
