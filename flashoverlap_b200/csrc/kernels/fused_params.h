// Parameter block of the persistent sm_100a GEMM(+collective)(+RMSNorm) kernel.
//
// One kernel covers what the reference spreads over a signalling GEMM, a
// counting kernel and a series of NCCL calls (reference: src/overlap_impl.cu:221-328,
// src/overlap/gemm_with_signal.h:127-202, src/overlap/gemm_with_scatter.h:127-197,
// src/wait.cuh:5-9).  The GEMM phase writes every finished tile where its
// consumer needs it (own memory or a peer's staging buffer) and bumps a counter
// per 128-row block on the owning GPU; the reduce phase, run by the
// communication warps of every CTA while the GEMM is still running (joined by
// the GEMM warps once they are out of tiles), waits (bounded) on those
// counters, sums the per-rank partials in fp32, optionally applies RMSNorm and
// writes the result locally (reduce-scatter) or to every peer (all-reduce).
#pragma once

#include <cuda.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define FO_HOST_DEVICE __host__ __device__
#else
#define FO_HOST_DEVICE
#endif

namespace fo {

constexpr int kMaxRanks = 8;

// CTA shape of the fused kernel: 8 GEMM warps (TMA, MMA, TMEM, signalling, 4 x
// epilogue) and one group of communication warps that reduces rows while the
// GEMM runs.  A row of the reduce phase is always handled by kGroupWarps warps.
constexpr int kGemmWarps = 8;
constexpr int kCommWarps = 4;
constexpr int kGroupWarps = 4;
constexpr int kFusedThreads = 32 * (kGemmWarps + kCommWarps);

// Layout of one counter set (32-bit words): arrival counters of the 128-row
// blocks, the all-reduce delivery counter, the per-source counters of a
// gathered A operand, the row-job counter of the reduce phase.
constexpr int kMaxTileRows = 2048;
constexpr int kFlagDone = kMaxTileRows;
constexpr int kFlagAReady = kMaxTileRows + 8;
constexpr int kFlagJob = kMaxTileRows + 32;
constexpr int kFlagWords = kMaxTileRows + 64;

// Rows up to this many values keep their RMSNorm weight vector in shared memory
// (and their sums in registers); wider rows take the two-pass path.
constexpr int kGammaSmemValues = 8192;

// Entries (uint64) per CTA of the optional phase trace.
constexpr int kTraceWords = 8;

// Where an element (row, col) of a logical row-major matrix lives in memory.
// tiled == 0: natural layout, offset = row * ld + col.
// tiled == 1: the reference's "reordered" layout (reference:
//   src/rmsnorm/rmsnorm.cuh:62-115, src/overlap/gemm_with_signal.h:148-165):
//   the matrix is cut into bm x bn tiles, tile t = (row/bm)*tn + col/bn lives in
//   slot s = ra[t]; with w = rldn*bn the element sits at
//   ((s / rldn) * bm + row % bm) * w + (s % rldn) * bn + col % bn.
//   With row_map (only with rldn == 1) the row index of that view goes through
//   the map first: the reference's scatter epilogue, which groups the rows of a
//   segment by (row % world) (reference: src/overlap/gemm_with_scatter.h:161-177).
struct OutLayout {
  int tiled;
  int bm, bn, tn, rldn;
  const int* ra;
  long long ld;
  const int* row_map;
};

enum OwnMode : int {
  OWN_SINGLE = 0,      // everything stays on this GPU (plain GEMM, TP = 1)
  OWN_BLOCK = 1,       // owner(row) = row / rows_per_owner (contiguous reduce-scatter)
  OWN_INTERLEAVE = 2,  // owner(row) = row % ws (all-reduce; reference-style reduce-scatter)
};

enum StatusCode : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT_PIPE = 1,    // an mbarrier inside the GEMM pipeline never completed
  ST_TIMEOUT_FLAG = 2,    // partials from some rank never arrived
  ST_TIMEOUT_DONE = 3,    // all-reduce results from some owner never arrived
  ST_BAD_INDEX = 4,       // an index array (reorder / row map) held an out-of-range entry
  ST_TIMEOUT_GATHER = 5,  // an all-gathered operand shard never arrived
};

// Written by the device on the first error only.  The word itself lives in
// device memory (the first error wins an atomic compare-and-swap there); the
// winner also copies the record into a mirror in mapped host memory, which the
// host reads without synchronising before every fused call.
struct StatusWord {
  uint32_t code;
  uint32_t rank;
  uint32_t where;  // role / unit that gave up
  uint32_t seen;   // counter value seen
  uint32_t want;   // counter value wanted
  uint32_t pad[3];
};

struct alignas(64) FusedParams {
  CUtensorMap tmA;  // A [M, K] row-major, box 64 x 128, 128-byte swizzle
  CUtensorMap tmB;  // B [N, K] row-major, box 64 x BN,  128-byte swizzle
  // All-gather -> GEMM: this rank's own rows [a_own_begin, a_own_end) of the
  // gathered A are read straight from the caller's shard through this map
  // (row 0 of the map = row a_own_begin), so they are never copied into the
  // gathered buffer.  a_own_end == a_own_begin: not used.
  CUtensorMap tmA_own;
  int a_own_begin, a_own_end;

  int M, N, K;
  int TM, TN;        // tile grid (BM = 128)
  int raster_group;  // tile rows walked column-major together (L2 reuse of B)
  int raster_taper;  // 1 = the last groups shrink by halves so that little is left to communicate after the last tile
  int force_full_grid;  // launch the requested number of CTAs even when there are fewer tiles
  int rot;           // first tile row of the walk (gathered operands start at the rank's own rows)
  int owner_stride;  // > 0 (block ownership): tile rows per owner; the walk then cycles through the owners
  int l2_hints;      // 1 = TMA loads carry L2 eviction hints (A panel kept, B panel streamed)

  // ---- GEMM epilogue destination -------------------------------------------
  int own_mode;             // OwnMode
  int ws, me;               // ranks in the group, this rank
  int rows_per_owner;       // M / ws
  void* epi_base[kMaxRanks];  // own_mode SINGLE: [0] = C; else staging slot of `me` on each owner
  OutLayout epi_layout;       // layout within the destination (tiled only with OWN_SINGLE)
  uint32_t* flag[kMaxRanks];  // per-owner arrival counters, one per tile row; null = no signalling

  // ---- reference-compatible signalling / tracing ----------------------------
  int* seg_counter;     // MM: per-segment tile counters (null = off)
  const int* cseg;      // device copy of tiles-per-segment
  int nseg;
  int* ticket_counter;  // monitor mode: global completion ticket (null = off)
  int* trace;           // monitor mode: trace[slot] = ticket
  const int* slot_of_tile;  // RA; null = identity

  // ---- A operand readiness (all-gather -> GEMM) -----------------------------
  const uint32_t* a_ready;  // per source-rank counter; null = A is ready at launch
  uint32_t a_ready_target;
  int a_src_end[kMaxRanks]; // source r contributed the rows [a_src_end[r-1], a_src_end[r]) of the gathered A
  // All-gather push (done by the communication warps of every CTA while the GEMM starts on this
  // rank's own shard): this rank's shard goes to every rank's gathered A.
  // (all-gather: the same shard to everybody; all-to-all dispatch: a different
  // block of rows, possibly empty, to every rank).
  int ag_push;                          // 0 = no push
  const void* ag_src[kMaxRanks];        // rows this rank sends to rank r
  long long ag_bytes[kMaxRanks];        // their size in bytes (multiple of 16, may be 0)
  void* ag_dst[kMaxRanks];       // where this rank's shard lives in rank r's gathered A
  uint32_t* ag_flag[kMaxRanks];  // rank r's a_ready counter for this rank
  // All-gather over NVLink SHARP (every rank receives the same rows): multicast
  // address of this rank's slot in the gathered A and of its a_ready counter;
  // one multimem.st per chunk then replaces the stores to every peer.  Null = peer-to-peer stores.
  void* ag_mc_dst;
  uint32_t* ag_mc_flag;

  // ---- reduce phase ---------------------------------------------------------
  int reduce;                      // 0 = kernel ends after the GEMM
  uint32_t* job_counter;           // next owned row to reduce (zero at launch); rows are claimed in order
  const void* stage;               // this GPU's staging: [ws][rows_per_owner][N]
  uint32_t flag_target;            // value every arrival counter must reach
  int norm;                        // apply RMSNorm after the sum
  const void* gamma;               // [N]
  float eps;
  int bcast;                       // 1 = write to every rank (all-reduce), 0 = only locally
  void* out[kMaxRanks];            // destination of reduced rows on each rank
  OutLayout out_layout;
  uint32_t* done[kMaxRanks];       // per-rank "rows delivered" counter (all-reduce)
  uint32_t done_target;

  // ---- NVLink SHARP mode -----------------------------------------------------
  // nvls == 1: the epilogue keeps the partial tiles in this GPU's own staging
  // buffer ([M][N], natural order, epi_base[0]); the owner of a row pulls the
  // sum over all ranks with multimem.ld_reduce, and an all-reduce result is
  // written to every rank with multimem.st.  The mc_* pointers are multicast
  // addresses of the staging buffer, arrival counters, result buffer and
  // delivery counter.
  int nvls;
  const void* mc_stage;
  uint32_t* mc_flag;
  void* mc_out;
  uint32_t* mc_done;

  // ---- phase trace ----------------------------------------------------------
  // Optional, kTraceWords x uint64 per CTA, times as %globaltimer nanoseconds:
  // [0] kernel start, [1] end of the GEMM phase, [2] last row reduced by this
  // CTA, [3] tiles computed, [4] first row reduced by this CTA (0 = none),
  // [5] rows reduced by this CTA, [6] all rows delivered (CTA 0 of an
  // all-reduce only), [7] unused.
  unsigned long long* phase_trace;
  // Optional row timeline of the reduce phase, 6 x M x uint64 (null = off), all
  // by the leading thread of the row group that claimed global row g: [g] row
  // claimed, [M + g] the row's stores issued, [2M + g] = CTA * 4 + row group,
  // [3M + g] the partials of all ranks were there, [4M + g] its chunks loaded
  // and summed, [5M + g] the group passed the row's barrier.
  unsigned long long* row_trace;

  // ---- failure reporting ----------------------------------------------------
  StatusWord* status;
  StatusWord* status_mirror;  // mapped host memory, may be null
  unsigned long long timeout_ns;
};

// Tile order: tile rows are walked in groups of `raster_group`; inside a group
// the walk is column-major so that one B panel serves the whole group from L2
// and tile rows still complete early and in order.  With `raster_taper` the
// last groups shrink (G, ..., G, G/2, G/4, ..., 1, 1): the rows of a group can
// only be reduced once the whole group is computed, so the size of the LAST
// group is what remains to be communicated after the last tile.
FO_HOST_DEVICE inline void tile_coords(const FusedParams& p, int t, int& m_blk, int& n_blk) {
  const int G = p.raster_group;
  int first = 0;      // first tile row of the group that holds tile t
  int rows_here = G;  // tile rows in that group
  int r = t;          // index of the tile inside the group
  if (!p.raster_taper) {
    const int per_group = G * p.TN;
    const int g = t / per_group;
    r = t - g * per_group;
    first = g * G;
    rows_here = (p.TM - first) < G ? (p.TM - first) : G;
  } else {
    // full groups while more than G tile rows remain, then halves
    int remaining = p.TM;
    int size = G;
    while (true) {
      if (remaining <= size) size = remaining > 1 ? (remaining + 1) / 2 : 1;
      const int tiles_here = size * p.TN;
      if (r < tiles_here || remaining == size) break;
      r -= tiles_here;
      first += size;
      remaining -= size;
    }
    rows_here = size;
  }
  int mb = first + r % rows_here;
  n_blk = r / rows_here;
  if (p.owner_stride > 0) {
    // Contiguous row ownership: position mb of the walk is tile row
    // (mb % ws) of ... every owner in turn, so that any stretch of the walk
    // sends to all owners alike and every owner's rows complete progressively
    // (walking owner by owner would complete an owner's rows only when the
    // LAST rank reaches its block, i.e. at the very end).  Each rank starts the
    // cycle at a different owner.
    const int o = (mb + p.me) % p.ws;
    mb = o * p.owner_stride + mb / p.ws;
  }
  m_blk = mb + p.rot;
  if (m_blk >= p.TM) m_blk -= p.TM;
}


}  // namespace fo
