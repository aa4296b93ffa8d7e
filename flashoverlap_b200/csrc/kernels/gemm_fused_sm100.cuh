// Persistent, warp-specialised sm_100a kernel: C = A * B^T on tcgen05 tensor
// cores with TMEM accumulators, operands staged by TMA, and the collective that
// follows the GEMM (all-reduce or reduce-scatter, optionally RMSNorm) fused in
// through peer-to-peer stores or NVLink SHARP (multimem) and system-scope
// counters.
//
// CTA layout (384 threads, one CTA per SM, grid <= number of SMs):
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads; with a
//                               gathered A operand it first waits for the source
//                               ranks whose rows the tile needs)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma / tcgen05.commit)
//   warp 2      TMEM allocator (allocates 2 x BN columns, frees them at the end)
//   warp 3      signalling     (one lane publishes finished tiles at system scope
//                               and bumps the owners' arrival counters)
//   warps 4-7   epilogue       (tcgen05.ld -> convert -> smem transpose ->
//                               coalesced 16-byte stores, local or to a peer)
//   warps 8-11  communication  (reduce phase: from the first cycle on they claim
//                               owned rows in completion order, wait (bounded)
//                               for the row's partials from every rank, sum them
//                               in fp32, apply RMSNorm and deliver the row;
//                               all-gather / all-to-all mode: they push this
//                               rank's rows of A to the other ranks)
// With CTAS == 2 two such CTAs form a cluster: both stage operands and run an
// epilogue for their own 128 rows, the MMA warp of rank 0 issues for the pair.
// After its last tile the eight GEMM warps of a CTA join the reduce phase as two
// more row groups, so the tail of the collective runs on every warp.
//
// Replaces, as one launch, the reference's signalling GEMM + wait kernel +
// segmented NCCL calls (reference: src/overlap_impl.cu:221-328): communication
// of finished rows runs under the computation of later tiles inside one kernel.
#pragma once

#include "fused_params.h"
#include "sm100_ptx.cuh"

namespace fo {

// CTAS == 1: one CTA computes a 128 x BN tile (tcgen05.mma.cta_group::1).
// CTAS == 2: a cluster of two CTAs computes a 256 x BN tile with
//   tcgen05.mma.cta_group::2; each CTA stages its own 128 rows of A and one
//   half of the B tile, so every SM fetches a third less per FLOP.
template <int BN_, int CTAS_ = 1, int BK_ = 64>
struct TileTraits {
  static constexpr int CTAS = CTAS_;
  static constexpr int BM = 128;           // rows per CTA
  static constexpr int TILE_M = BM * CTAS;  // rows per tile
  static constexpr int BN = BN_;
  static constexpr int BK = BK_;       // K depth of one pipeline stage
  static constexpr int ATOM_K = 64;    // 64 x 2 bytes = one 128-byte swizzle row; one TMA box
  static constexpr int ATOMS = BK / ATOM_K;
  static constexpr int UMMA_K = 16;
  static constexpr int A_ATOM_BYTES = BM * ATOM_K * 2;
  static constexpr int A_BYTES = A_ATOM_BYTES * ATOMS;
  static constexpr int B_ROWS = BN / CTAS;  // rows of B staged by each CTA
  static constexpr int B_ATOM_BYTES = B_ROWS * ATOM_K * 2;
  static constexpr int B_BYTES = B_ATOM_BYTES * ATOMS;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_WARPS = 4;
  static constexpr int EPI_SLAB_BYTES = 32 * 128;  // 32 rows x 64 columns of 16-bit values
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_SLAB_BYTES;
  static constexpr int BAR_BYTES = 512;
  static constexpr int GAMMA_BYTES = kGammaSmemValues * 2;  // RMSNorm weight vector of rows up to 8192 values
  static constexpr int SMEM_LIMIT = 227 * 1024;
  static constexpr int STAGES_RAW = (SMEM_LIMIT - 1024 - EPI_BYTES - BAR_BYTES - GAMMA_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + GAMMA_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulator buffers; power of two >= 32
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
  static_assert(CTAS == 1 || CTAS == 2, "one CTA or a CTA pair");
  static_assert(BK == 64 || BK == 128, "BK must be 64 or 128");
  static_assert(STAGES >= 3, "pipeline too shallow");
};

constexpr int kThreads = kFusedThreads;  // 8 GEMM warps + 4 communication warps
constexpr int kGemmThreads = 32 * kGemmWarps;

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ long long layout_offset(const OutLayout& L, int row, int col) {
  if (!L.tiled) return static_cast<long long>(row) * L.ld + col;
  const int t = (row / L.bm) * L.tn + col / L.bn;
  const int s = L.ra ? L.ra[t] : t;
  const long long w = static_cast<long long>(L.rldn) * L.bn;
  long long view_row = static_cast<long long>(s / L.rldn) * L.bm + row % L.bm;
  if (L.row_map != nullptr) view_row = L.row_map[view_row];
  return view_row * w + (s % L.rldn) * L.bn + col % L.bn;
}

__device__ __forceinline__ void report_error(StatusWord* st, StatusWord* mirror, uint32_t code, uint32_t rank,
                                             uint32_t where, uint32_t seen, uint32_t want) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->rank = rank;
    st->where = where;
    st->seen = seen;
    st->want = want;
    if (mirror != nullptr) {  // details first, the code last: a host that sees the code sees the rest
      volatile StatusWord* m = mirror;
      m->rank = rank;
      m->where = where;
      m->seen = seen;
      m->want = want;
      __threadfence_system();
      m->code = code;
    }
    __threadfence_system();
  }
}
__device__ __forceinline__ void report_error(const FusedParams& p, uint32_t code, uint32_t where, uint32_t seen,
                                             uint32_t want) {
  report_error(p.status, p.status_mirror, code, static_cast<uint32_t>(p.me), where, seen, want);
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// y = round16(x * rstd) * w, both steps rounded to the 16-bit type, which is
// the reference's rounding order (reference: src/rmsnorm/rmsnorm.cuh:107-111).
template <bool BF16>
__device__ __forceinline__ uint32_t norm_pack2(float a, float b, float rstd, uint32_t w2) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a * rstd, b * rstd);
    __nv_bfloat162 r = __hmul2(v, *reinterpret_cast<__nv_bfloat162*>(&w2));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __half2 v = __floats2half2_rn(a * rstd, b * rstd);
    __half2 r = __hmul2(v, *reinterpret_cast<__half2*>(&w2));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

// ---------------------------------------------------------------------------
// reduce phase: groups of kGroupWarps warps, one owned row at a time
// ---------------------------------------------------------------------------
// Shared-memory scratch of one row group (double-buffered by iteration parity:
// one barrier per row then orders both the next-row broadcast and the exchange
// of the partial sums of squares).
struct GroupScratch {
  uint32_t job[2];
  float ssq[2][kGroupWarps];
};

__device__ __forceinline__ void group_barrier(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kGroupWarps * 32) : "memory");
}

// Rows this rank owns are numbered lr = 0 .. rows_per_owner-1 in the order in
// which the GEMM phase completes their tile rows (ascending: the raster walks
// tile rows upwards from p.rot, and a rank's block is the last one it computes).
// Every group claims the next row from a counter in global memory, so rows are
// always taken in completion order by whichever warps are free: the
// communication warps from the start, the GEMM warps once their tiles are done.
// For one row the group waits (bounded) until the partials of every rank have
// arrived, sums them in fp32 and rounds the sum to the 16-bit type (the value an
// all-reduce would have produced).  Rows of up to 8192 values stay in registers
// (8 x 16 bytes per thread) between the sum and the RMSNorm scaling; wider rows
// take two passes (the rounded sums are parked in this rank's output row and read
// back).  With a single source per chunk (one rank, or NVLS) the loads of the
// next row are issued before the current row is scaled and stored, if that
// row's partials have already arrived.  NVLS == true replaces the per-rank
// loads by one multimem.ld_reduce per chunk and the per-rank result stores by
// one multimem.st.  WS > 0 fixes the number of ranks at compile time; WS == 0
// is the generic fallback.
// (Inlined into the kernel, which calls it from a single place: the parameter
// block must stay a kernel parameter read through the constant bank.  Behind a
// function call it would be read through a generic pointer, one global load per
// field access, which made every row several times slower.)
template <bool BF16, int WS, bool NVLS>
__device__ __forceinline__ void comm_worker(const FusedParams& p, GroupScratch* gs, uint32_t gamma_smem, int group,
                                            int wg, int lane, uint64_t deadline, volatile uint32_t* abort_flag) {
  constexpr int BM = 128;
  constexpr int GT = kGroupWarps * 32;  // threads per row
  constexpr int CPT = 8;                // 16-byte chunks per thread held in registers
  constexpr bool GENERIC = !NVLS && WS == 0;  // any number of ranks: sources are added one after the other
  constexpr int NS = (NVLS || GENERIC) ? 1 : WS;
  constexpr int BATCH = NS >= CPT ? 1 : CPT / NS;  // chunks loaded together
  const int ws = p.ws;
  const int nsrc = NVLS ? 1 : ws;
  const int n_chunks = p.N >> 3;
  const bool one_pass = n_chunks <= GT * CPT;
  const int last_chunk = n_chunks - 1;
  const int tid = wg * 32 + lane;
  const int rows_local = p.rows_per_owner;
  const uint16_t* stage = reinterpret_cast<const uint16_t*>(p.stage);
  const long long src_stride = static_cast<long long>(rows_local) * p.N;
  const uint32_t* my_flag = p.flag[p.me];
  const uint4* gamma = reinterpret_cast<const uint4*>(p.gamma);
  const bool leader = wg == 0 && lane == 0;
  unsigned long long t_first = 0, t_last = 0;
  uint32_t rows_done = 0;

  auto store_out = [&](int out_row, int c, const uint4& o) {
    const long long off = layout_offset(p.out_layout, out_row, c * 8);
    if (NVLS && p.bcast) {
      ptx::multimem_st_v4(reinterpret_cast<uint16_t*>(p.mc_out) + off, o);  // lands on every rank
    } else if (p.bcast) {
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < ws) {
          int d = p.me + 1 + r;  // start with the next rank: owners spread over destinations
          if (d >= ws) d -= ws;
          ptx::st_v4(reinterpret_cast<uint16_t*>(p.out[d]) + off, o);
        }
      }
    } else {
      ptx::st_v4(reinterpret_cast<uint16_t*>(p.out[p.me]) + off, o);
    }
  };
  auto sum_sources = [&](const uint4 (&v)[NS]) -> uint4 {
    if constexpr (NVLS || WS == 1) {
      return v[0];  // NVLS: summed by the switch in fp32, rounded once; one rank: nothing to add
    } else {
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = 0.f;
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) {  // NS is the number of ranks here
        float2 f;
        f = unpack2<BF16>(v[sidx].x); a[0] += f.x; a[1] += f.y;
        f = unpack2<BF16>(v[sidx].y); a[2] += f.x; a[3] += f.y;
        f = unpack2<BF16>(v[sidx].z); a[4] += f.x; a[5] += f.y;
        f = unpack2<BF16>(v[sidx].w); a[6] += f.x; a[7] += f.y;
      }
      uint4 h;
      h.x = pack2<BF16>(a[0], a[1]);
      h.y = pack2<BF16>(a[2], a[3]);
      h.z = pack2<BF16>(a[4], a[5]);
      h.w = pack2<BF16>(a[6], a[7]);
      return h;
    }
  };
  auto sq = [&](const uint4& h) -> float {
    float2 f;
    float r;
    f = unpack2<BF16>(h.x); r = f.x * f.x + f.y * f.y;
    f = unpack2<BF16>(h.y); r += f.x * f.x + f.y * f.y;
    f = unpack2<BF16>(h.z); r += f.x * f.x + f.y * f.y;
    f = unpack2<BF16>(h.w); r += f.x * f.x + f.y * f.y;
    return r;
  };
  auto scale = [&](const uint4& h, float rstd, const uint4& w) -> uint4 {
    float2 f;
    uint4 o;
    f = unpack2<BF16>(h.x); o.x = norm_pack2<BF16>(f.x, f.y, rstd, w.x);
    f = unpack2<BF16>(h.y); o.y = norm_pack2<BF16>(f.x, f.y, rstd, w.y);
    f = unpack2<BF16>(h.z); o.z = norm_pack2<BF16>(f.x, f.y, rstd, w.z);
    f = unpack2<BF16>(h.w); o.w = norm_pack2<BF16>(f.x, f.y, rstd, w.w);
    return o;
  };
  // where owned row lr lives: global row, 128-row block, partial rows, output row
  auto global_row = [&](int lr) -> int {
    if (p.own_mode == OWN_BLOCK) return p.me * rows_local + lr;
    if (p.own_mode == OWN_INTERLEAVE) return lr * ws + p.me;
    return lr;
  };
  auto partials_of = [&](int lr, int g) -> const uint16_t* {
    // NVLS: partials sit at their global row in every rank's staging buffer
    return NVLS ? reinterpret_cast<const uint16_t*>(p.mc_stage) + static_cast<long long>(g) * p.N
                : stage + static_cast<long long>(lr) * p.N;
  };
  auto load_chunk = [&](uint4 (&v)[NS], const uint16_t* src0, int c) {
#pragma unroll
    for (int sidx = 0; sidx < NS; ++sidx) {
      if (sidx < nsrc) {
        if constexpr (NVLS) v[sidx] = ptx::multimem_ld_reduce_add_v4<BF16>(src0 + c * 8);
        else v[sidx] = ptx::ld_cg_v4(src0 + sidx * src_stride + c * 8);
      }
    }
  };
  // generic world size: one chunk summed over all ranks, four loads in flight at a time
  auto load_sum_generic = [&](const uint16_t* src0, int c) -> uint4 {
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
    for (int s0 = 0; s0 < ws; s0 += 4) {
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (s0 + k < ws) v[k] = ptx::ld_cg_v4(src0 + (s0 + k) * src_stride + c * 8);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (s0 + k < ws) {
          float2 f;
          f = unpack2<BF16>(v[k].x); a[0] += f.x; a[1] += f.y;
          f = unpack2<BF16>(v[k].y); a[2] += f.x; a[3] += f.y;
          f = unpack2<BF16>(v[k].z); a[4] += f.x; a[5] += f.y;
          f = unpack2<BF16>(v[k].w); a[6] += f.x; a[7] += f.y;
        }
      }
    }
    uint4 h;
    h.x = pack2<BF16>(a[0], a[1]);
    h.y = pack2<BF16>(a[2], a[3]);
    h.z = pack2<BF16>(a[4], a[5]);
    h.w = pack2<BF16>(a[6], a[7]);
    return h;
  };
  int ready_rb = -1;  // last 128-row block this warp has seen complete (rows are claimed in ascending order)
  // Bounded wait until every rank's partials for block rb have arrived (0 on timeout).
  auto wait_block = [&](int rb) -> uint32_t {
    if (rb == ready_rb) return 1u;
    uint32_t ok = 1;
    if (lane == 0) {
      uint32_t seen = 0;
      if (!ptx::wait_counter_geq(my_flag + rb, p.flag_target, deadline, &seen)) {
        report_error(p, ST_TIMEOUT_FLAG, rb, seen, p.flag_target);
        *abort_flag = 1;
        ok = 0;
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();  // lane 0's acquire is ordered before the other lanes' loads of the partials
    if (ok) ready_rb = rb;
    return ok;
  };
  // One look at the counter, no waiting.
  auto block_ready_now = [&](int rb) -> bool {
    if (rb == ready_rb) return true;
    uint32_t ok = 0;
    if (lane == 0) ok = static_cast<int32_t>(ptx::ld_acquire_sys(my_flag + rb) - p.flag_target) >= 0 ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    if (ok) ready_rb = rb;
    return ok != 0;
  };

  // the first row, and the claim of the one after it
  uint32_t claimed = 0;
  if (leader) {
    gs->job[0] = atomicAdd(p.job_counter, 1u);
    claimed = atomicAdd(p.job_counter, 1u);
  }
  group_barrier(group);
  int lr = static_cast<int>(gs->job[0]);
  constexpr uint32_t kDeliveryBatch = 4;
  uint32_t undelivered = 0;  // rows this warp has stored but not yet counted on the delivery counters
  const bool timeline = p.row_trace != nullptr && leader;
  constexpr bool PREFETCH = NS == 1 && !GENERIC;  // a second register set for the next row fits
  bool have = false;  // `pre` holds the chunks of row lr, requested during the previous iteration
  uint4 pre[PREFETCH ? CPT : 1];

  for (int it = 0; lr < rows_local; ++it) {
    const int par = it & 1;
    const int g = global_row(lr);
    const int out_row = p.bcast ? g : lr;
    const uint16_t* src0 = partials_of(lr, g);
    const unsigned long long t_claim = timeline ? ptx::globaltimer_ns() : 0ull;
    const uint32_t ok = have ? 1u : wait_block(g / BM);
    const unsigned long long t_ready = timeline ? ptx::globaltimer_ns() : 0ull;

    // ---- sum of the partial rows (and the sum of squares) ----
    uint4 h[CPT];
    float ssq = 0.f;
    uint16_t* park = reinterpret_cast<uint16_t*>(p.out[p.me]);  // wide rows only
    if (ok && one_pass) {
      if constexpr (GENERIC) {
#pragma unroll
        for (int u = 0; u < CPT; ++u) {
          const int c = u * GT + tid;
          if (c < n_chunks) {
            h[u] = load_sum_generic(src0, c);
            if (p.norm) ssq += sq(h[u]);
            else store_out(out_row, c, h[u]);
          }
        }
      } else if constexpr (NS == 1) {
        // One source per chunk: all loads of the row go out back to back.  They
        // are unconditional (a chunk index past the end of the row is clamped,
        // the value ignored): a load inside a conditional block together with
        // an instruction that uses its value waits for the load before it.
        if (have) {
#pragma unroll
          for (int u = 0; u < CPT; ++u) h[u] = pre[PREFETCH ? u : 0];
        } else {
#pragma unroll
          for (int u = 0; u < CPT; ++u) {
            const int c = min(u * GT + tid, last_chunk);
            if constexpr (NVLS) h[u] = ptx::multimem_ld_reduce_add_v4<BF16>(src0 + c * 8);
            else h[u] = ptx::ld_cg_v4(src0 + c * 8);
          }
        }
#pragma unroll
        for (int u = 0; u < CPT; ++u) {
          const int c = u * GT + tid;
          if (p.norm) ssq += c < n_chunks ? sq(h[u]) : 0.f;
          else if (c < n_chunks) store_out(out_row, c, h[u]);
        }
      } else {
        // Software pipeline over batches of chunks: the loads of batch k+1 are in
        // flight while batch k is summed.  Two register sets alternate by the
        // (compile-time) batch index, so nothing is copied; the loads are
        // unconditional (a chunk index past the row's end is clamped and its
        // value ignored), so that they form straight-line code and all go out
        // before the first use.
        constexpr int NB = CPT / BATCH;
        uint4 buf[2][BATCH][NS];
        auto issue = [&](int k, uint4 (&dst)[BATCH][NS]) {
#pragma unroll
          for (int u = 0; u < BATCH; ++u) {
            const int c = min((k * BATCH + u) * GT + tid, last_chunk);
#pragma unroll
            for (int sidx = 0; sidx < NS; ++sidx) dst[u][sidx] = ptx::ld_cg_v4(src0 + sidx * src_stride + c * 8);
          }
        };
        issue(0, buf[0]);
#pragma unroll
        for (int k = 0; k < NB; ++k) {
          if (k + 1 < NB) issue(k + 1, buf[(k + 1) & 1]);
#pragma unroll
          for (int u = 0; u < BATCH; ++u) {
            const int c = (k * BATCH + u) * GT + tid;
            h[k * BATCH + u] = sum_sources(buf[k & 1][u]);
            if (p.norm) ssq += c < n_chunks ? sq(h[k * BATCH + u]) : 0.f;
            else if (c < n_chunks) store_out(out_row, c, h[k * BATCH + u]);
          }
        }
      }
    } else if (ok) {
      // wide rows: first pass sums and parks the rounded sums in this rank's output row
      for (int c = tid; c < n_chunks; c += GT) {
        uint4 hv;
        if constexpr (GENERIC) {
          hv = load_sum_generic(src0, c);
        } else {
          uint4 v[NS];
          load_chunk(v, src0, c);
          hv = sum_sources(v);
        }
        if (p.norm) {
          ssq += sq(hv);
          ptx::st_v4(park + layout_offset(p.out_layout, out_row, c * 8), hv);
        } else {
          store_out(out_row, c, hv);
        }
      }
    }
    const unsigned long long t_sum = timeline ? ptx::globaltimer_ns() : 0ull;

    // ---- one barrier: exchange the partial sums of squares, learn the next row ----
    if (p.norm) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if (lane == 0) gs->ssq[par][wg] = ssq;
    }
    if (leader) gs->job[par ^ 1] = claimed;
    group_barrier(group);
    const int next_lr = static_cast<int>(gs->job[par ^ 1]);
    if (leader && next_lr < rows_local) claimed = atomicAdd(p.job_counter, 1u);  // its latency hides behind the stores
    if (p.norm) {
      ssq = 0.f;
#pragma unroll
      for (int w = 0; w < kGroupWarps; ++w) ssq += gs->ssq[par][w];
    }
    const unsigned long long t_bar = timeline ? ptx::globaltimer_ns() : 0ull;

    // ---- the next row's loads go out before this row is scaled and stored, if its partials are there ----
    have = false;
    if constexpr (PREFETCH) {
      if (one_pass && next_lr < rows_local) {
        const int g2 = global_row(next_lr);
        if (block_ready_now(g2 / BM)) {
          const uint16_t* src2 = partials_of(next_lr, g2);
#pragma unroll
          for (int u = 0; u < CPT; ++u) {
            const int c = min(u * GT + tid, last_chunk);
            if constexpr (NVLS) pre[u] = ptx::multimem_ld_reduce_add_v4<BF16>(src2 + c * 8);
            else pre[u] = ptx::ld_cg_v4(src2 + c * 8);
          }
          have = true;
        }
      }
    }

    // ---- RMSNorm scaling and delivery of this row ----
    if (p.norm && ok) {
      const float rstd = rsqrtf(ssq / static_cast<float>(p.N) + p.eps);
      if (one_pass) {
#pragma unroll
        for (int u = 0; u < CPT; ++u) {
          const int c = u * GT + tid;
          if (c < n_chunks) {
            store_out(out_row, c, scale(h[u], rstd, ptx::ld_shared_v4(gamma_smem + (static_cast<uint32_t>(c) << 4))));
          }
        }
      } else {
        for (int c = tid; c < n_chunks; c += GT) {  // every thread re-reads exactly the chunks it wrote
          const uint4 hv = ptx::ld_cg_v4(park + layout_offset(p.out_layout, out_row, c * 8));
          const uint4 wv = __ldg(gamma + c);
          store_out(out_row, c, scale(hv, rstd, wv));
        }
      }
    }
    // Delivery counts are only read at the end of the kernel, and a release
    // at system scope waits for this warp's stores to be acknowledged by the
    // peers: signal a batch of rows at a time.
    if (ok && p.bcast) ++undelivered;
    if (undelivered != 0 && (undelivered == kDeliveryBatch || next_lr >= rows_local)) {
      __syncwarp();  // every lane's stores of these row parts precede the releases below
      if constexpr (NVLS) {
        if (lane == 0) ptx::multimem_red_release_add(p.mc_done, undelivered);
      } else {
        if (lane < ws && p.done[lane] != nullptr) ptx::red_release_sys_add(p.done[lane], undelivered);
      }
      undelivered = 0;
    }
    if (ok && timeline) {
      const long long m = p.M;
      p.row_trace[g] = t_claim;
      p.row_trace[m + g] = ptx::globaltimer_ns();
      p.row_trace[2 * m + g] = static_cast<unsigned long long>(blockIdx.x) * 4ull + group;
      p.row_trace[3 * m + g] = t_ready;
      p.row_trace[4 * m + g] = t_sum;
      p.row_trace[5 * m + g] = t_bar;
    }
    if (ok && p.phase_trace != nullptr && leader) {
      t_last = ptx::globaltimer_ns();
      if (t_first == 0) t_first = t_last;
      ++rows_done;
    }
    lr = next_lr;
  }
  if (p.phase_trace != nullptr && leader && rows_done != 0) {
    unsigned long long* tr = p.phase_trace + static_cast<unsigned long long>(kTraceWords) * blockIdx.x;
    atomicMax(tr + 2, t_last);
    atomicMin(tr + 4, t_first);
    atomicAdd(tr + 5, static_cast<unsigned long long>(rows_done));
  }
}

template <bool BF16>
__device__ __forceinline__ void comm_dispatch(const FusedParams& p, GroupScratch* gs, uint32_t gamma_smem, int group, int wg,
                                           int lane, uint64_t deadline, volatile uint32_t* abort_flag) {
  if (p.nvls) {
    comm_worker<BF16, 1, true>(p, gs, gamma_smem, group, wg, lane, deadline, abort_flag);
    return;
  }
  switch (p.ws) {
    case 1: comm_worker<BF16, 1, false>(p, gs, gamma_smem, group, wg, lane, deadline, abort_flag); break;
    case 2: comm_worker<BF16, 2, false>(p, gs, gamma_smem, group, wg, lane, deadline, abort_flag); break;
    case 4: comm_worker<BF16, 4, false>(p, gs, gamma_smem, group, wg, lane, deadline, abort_flag); break;
    case 8: comm_worker<BF16, 8, false>(p, gs, gamma_smem, group, wg, lane, deadline, abort_flag); break;
    default: comm_worker<BF16, 0, false>(p, gs, gamma_smem, group, wg, lane, deadline, abort_flag); break;
  }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int BN, int BK_, bool BF16, int CTAS>
__global__ void __launch_bounds__(kThreads, 1) gemm_fused_sm100_kernel(const __grid_constant__ FusedParams p) {
  using T = TileTraits<BN, CTAS, BK_>;
  constexpr int BM = T::BM, BK = T::BK, STAGES = T::STAGES, TILE_M = T::TILE_M;
  // rank inside the CTA pair; rank 0 (the leader) issues the MMAs of the pair
  const uint32_t cta_rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;
  const int first_tile = static_cast<int>(blockIdx.x) / CTAS;
  const int tile_stride = static_cast<int>(gridDim.x) / CTAS;

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle of TMA and UMMA.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * T::A_BYTES;
  uint8_t* smem_epi = smem + STAGES * T::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + T::EPI_BYTES);
  const uint32_t gamma_smem = ptx::smem_u32(smem_epi + T::EPI_BYTES + T::BAR_BYTES);  // [N] RMSNorm weights
  uint64_t* full_bar = bars;                   // [STAGES] TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;         // [STAGES] MMA -> TMA
  uint64_t* tfull_bar = bars + 2 * STAGES;     // [2] MMA -> epilogue
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* epi_prog = tmem_slot + 4;  // [4] tiles finished by each epilogue warp
  uint64_t* pair_bar = bars + 2 * STAGES + 8;  // teardown handshake between the CTAs of a pair
  GroupScratch* group_scratch = reinterpret_cast<GroupScratch*>(bars + 40);  // [3] row groups of the reduce phase

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t t_start = ptx::globaltimer_ns();
  const uint64_t deadline = t_start + p.timeout_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], T::EPI_WARPS * CTAS);  // the leader hears from both epilogues
    }
    ptx::mbar_init(pair_bar, 1);
    *abort_flag = 0;
    for (int i = 0; i < 4; ++i) epi_prog[i] = 0;
    if (p.phase_trace != nullptr) {
      unsigned long long* tr = p.phase_trace + static_cast<unsigned long long>(kTraceWords) * blockIdx.x;
      tr[0] = t_start;
      tr[1] = tr[2] = tr[3] = tr[5] = tr[6] = tr[7] = 0;
      tr[4] = ~0ull;
    }
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (p.reduce && p.norm && p.N <= kGammaSmemValues) {
    // the RMSNorm weights, once per CTA: every row group reads them for every row
    const uint4* gamma = reinterpret_cast<const uint4*>(p.gamma);
    for (int c = threadIdx.x; c < (p.N >> 3); c += kThreads) {
      ptx::st_shared_v4(gamma_smem + (static_cast<uint32_t>(c) << 4), __ldg(gamma + c));
    }
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&p.tmA);
    ptx::prefetch_tensormap(&p.tmB);
    if (p.a_own_end > p.a_own_begin) ptx::prefetch_tensormap(&p.tmA_own);
  }
  if (warp == 2) {
    if constexpr (CTAS == 2) {
      ptx::tmem_alloc_pair(tmem_slot, T::TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, T::TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (CTAS == 2) ptx::cluster_sync();  // both CTAs' barriers exist before anyone signals across
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.TM * p.TN;
  const int num_kb = (p.K + BK - 1) / BK;  // a K tail is zero-filled by TMA

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // A row panel serves every tile of its raster group (kept in L2), a B
      // panel is read by the group's tiles at about the same time and then
      // not again before the next group (dropped first).
      const uint64_t pol_a = ptx::l2_policy_evict_last();
      const uint64_t pol_b = ptx::l2_policy_evict_first();
      const int own_begin = p.me == 0 ? 0 : p.a_src_end[p.me - 1];  // gathered A: this rank's own rows
      const int own_end = p.a_src_end[p.me];
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
        int m_blk, n_blk;
        tile_coords(p, t, m_blk, n_blk);
        const int a_row = m_blk * TILE_M + static_cast<int>(cta_rank) * BM;
        const int b_row = n_blk * BN + static_cast<int>(cta_rank) * T::B_ROWS;
        // this CTA's 128 rows of A come from the caller's own shard (never copied) or from the (gathered) A
        const bool own_rows = a_row >= p.a_own_begin && a_row + BM <= p.a_own_end;
        const CUtensorMap* map_a = own_rows ? &p.tmA_own : &p.tmA;
        const int a_row_map = own_rows ? a_row - p.a_own_begin : a_row;
        if (p.a_ready != nullptr && !own_rows) {
          // Gathered A: wait until every source rank whose rows overlap
          // [a_row, a_row + BM) has delivered them into local memory, then order
          // those generic-proxy writes before the async-proxy (TMA) reads.
          for (int r = 0; r < p.ws && ok; ++r) {
            const int r_begin = r == 0 ? 0 : p.a_src_end[r - 1];
            const int r_end = p.a_src_end[r];
            if (r_end <= r_begin || r_end <= a_row || r_begin >= a_row + BM) continue;
            uint32_t seen = 0;
            if (!ptx::wait_counter_geq(p.a_ready + r, p.a_ready_target, deadline, &seen)) {
              report_error(p, ST_TIMEOUT_GATHER, r, seen, p.a_ready_target);
              *abort_flag = 1;
              ok = false;
            }
          }
          if (!ok) break;
          ptx::fence_proxy_async_all();
          if (p.phase_trace != nullptr && (a_row < own_begin || a_row >= own_end)) {
            // first tile of this CTA that needed rows of another rank: when it could start
            unsigned long long* tr = p.phase_trace + static_cast<unsigned long long>(kTraceWords) * blockIdx.x;
            if (tr[4] == ~0ull) tr[4] = ptx::globaltimer_ns();
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, deadline)) {
            report_error(p, ST_TIMEOUT_PIPE, 0x100u + stage, kb, t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if constexpr (CTAS == 2) {
            // both CTAs' bytes are counted on the leader's barrier
            if (cta_rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * T::STAGE_BYTES);
#pragma unroll
            for (int h = 0; h < T::ATOMS; ++h) {  // one box of 64 K-values per swizzle atom
              if (p.l2_hints) {
                ptx::tma_load_2d_pair_hint(smem_a + stage * T::A_BYTES + h * T::A_ATOM_BYTES, map_a, &full_bar[stage],
                                           kb * BK + h * T::ATOM_K, a_row_map, pol_a);
                ptx::tma_load_2d_pair_hint(smem_b + stage * T::B_BYTES + h * T::B_ATOM_BYTES, &p.tmB, &full_bar[stage],
                                           kb * BK + h * T::ATOM_K, b_row, pol_b);
              } else {
                ptx::tma_load_2d_pair(smem_a + stage * T::A_BYTES + h * T::A_ATOM_BYTES, map_a, &full_bar[stage],
                                      kb * BK + h * T::ATOM_K, a_row_map);
                ptx::tma_load_2d_pair(smem_b + stage * T::B_BYTES + h * T::B_ATOM_BYTES, &p.tmB, &full_bar[stage],
                                      kb * BK + h * T::ATOM_K, b_row);
              }
            }
          } else {
            ptx::mbar_arrive_expect_tx(&full_bar[stage], T::STAGE_BYTES);
#pragma unroll
            for (int h = 0; h < T::ATOMS; ++h) {
              if (p.l2_hints) {
                ptx::tma_load_2d_hint(smem_a + stage * T::A_BYTES + h * T::A_ATOM_BYTES, map_a, &full_bar[stage],
                                      kb * BK + h * T::ATOM_K, a_row_map, pol_a);
                ptx::tma_load_2d_hint(smem_b + stage * T::B_BYTES + h * T::B_ATOM_BYTES, &p.tmB, &full_bar[stage],
                                      kb * BK + h * T::ATOM_K, b_row, pol_b);
              } else {
                ptx::tma_load_2d(smem_a + stage * T::A_BYTES + h * T::A_ATOM_BYTES, map_a, &full_bar[stage],
                                 kb * BK + h * T::ATOM_K, a_row_map);
                ptx::tma_load_2d(smem_b + stage * T::B_BYTES + h * T::B_ATOM_BYTES, &p.tmB, &full_bar[stage],
                                 kb * BK + h * T::ATOM_K, b_row);
              }
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (ok && p.a_ready != nullptr && blockIdx.x == 0) {
        // The kernel may only end when every rank's pushes of this call have
        // arrived, also those of ranks that sent this rank no rows: it keeps a
        // rank from running more than one call ahead of a peer, which is what
        // makes two alternating buffer and counter sets sufficient.
        for (int r = 0; r < p.ws; ++r) {
          uint32_t seen = 0;
          if (!ptx::wait_counter_geq(p.a_ready + r, p.a_ready_target, deadline, &seen)) {
            report_error(p, ST_TIMEOUT_GATHER, 0x100u + r, seen, p.a_ready_target);
            break;
          }
        }
      }
      if (!ok) {
        // Give copies that are still in flight time to land before the CTA
        // releases its shared memory.
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(BF16 ? 1 : 0, TILE_M, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride, ++it) {
        const int buf = it & 1;
        const uint32_t use = static_cast<uint32_t>(it >> 1);
        if (!ptx::mbar_wait(&tempty_bar[buf], (use & 1u) ^ 1u, deadline)) {
          report_error(p, ST_TIMEOUT_PIPE, 0x200u + buf, it, t);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, deadline)) {
            report_error(p, ST_TIMEOUT_PIPE, 0x300u + stage, kb, t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int h = 0; h < T::ATOMS; ++h) {
            const uint64_t da =
                ptx::make_smem_desc_k_sw128(ptx::smem_u32(smem_a + stage * T::A_BYTES + h * T::A_ATOM_BYTES));
            const uint64_t db =
                ptx::make_smem_desc_k_sw128(ptx::smem_u32(smem_b + stage * T::B_BYTES + h * T::B_ATOM_BYTES));
#pragma unroll
            for (int k = 0; k < T::ATOM_K / T::UMMA_K; ++k) {
              // advancing K by 16 elements = 32 bytes = 2 descriptor address units
              const uint32_t acc = (kb | h | k) != 0 ? 1u : 0u;
              if constexpr (CTAS == 2) ptx::umma_f16_ss_pair(d_tmem, da + 2u * k, db + 2u * k, idesc, acc);
              else ptx::umma_f16_ss(d_tmem, da + 2u * k, db + 2u * k, idesc, acc);
            }
          }
          // frees the stage (in both CTAs of a pair) once the MMAs have read it
          if constexpr (CTAS == 2) ptx::umma_commit_pair(&empty_bar[stage], 3);
          else ptx::umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {  // accumulator complete
          if constexpr (CTAS == 2) ptx::umma_commit_pair(&tfull_bar[buf], 3);
          else ptx::umma_commit(&tfull_bar[buf]);
        }
      }
    }
  } else if (warp >= 4 && warp < kGemmWarps) {
    // ===================== epilogue =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t slab = ptx::smem_u32(smem_epi + q * T::EPI_SLAB_BYTES);
    int it = 0;
    bool ok = true;
    // the accumulator-free barrier lives in the leader CTA of a pair
    const uint32_t tempty_addr0 = CTAS == 2 ? ptx::mapa_shared(ptx::smem_u32(&tempty_bar[0]), 0) : 0u;
    for (int t = first_tile; t < num_tiles && ok; t += tile_stride, ++it) {
      int m_blk, n_blk;
      tile_coords(p, t, m_blk, n_blk);
      const int buf = it & 1;
      const uint32_t use = static_cast<uint32_t>(it >> 1);
      if (!ptx::mbar_wait(&tfull_bar[buf], use & 1u, deadline)) {
        if (lane == 0) {
          report_error(p, ST_TIMEOUT_PIPE, 0x400u + buf, it, t);
          *abort_flag = 1;
        }
        ok = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * BN);
      const int row0 = m_blk * TILE_M + static_cast<int>(cta_rank) * BM + q * 32;  // first global row of this warp's slab

#pragma unroll 1
      for (int cc = 0; cc < BN / 64; ++cc) {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld_32x32b_x32(t_row + cc * 64, r0);
        ptx::tmem_ld_32x32b_x32(t_row + cc * 64 + 32, r1);
        ptx::tmem_ld_wait();
        if (cc == BN / 64 - 1) {
          // accumulator fully read: hand the TMEM buffer back to the MMA warp
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(tempty_addr0 + 8u * buf);
            else ptx::mbar_arrive(&tempty_bar[buf]);
          }
        }
        // registers -> swizzled smem slab (row = lane, 8 chunks of 16 bytes)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack2<BF16>(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
          v.y = pack2<BF16>(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
          v.z = pack2<BF16>(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
          v.w = pack2<BF16>(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
          ptx::st_shared_v4(slab + lane * 128 + ((j ^ (lane & 7)) << 4), v);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack2<BF16>(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
          v.y = pack2<BF16>(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
          v.z = pack2<BF16>(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
          v.w = pack2<BF16>(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
          ptx::st_shared_v4(slab + lane * 128 + (((j + 4) ^ (lane & 7)) << 4), v);
        }
        __syncwarp();
        // smem slab -> global: 8 lanes cover one 128-byte row segment
        const int chunk = lane & 7;
        const int col = n_blk * BN + cc * 64 + chunk * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          const uint4 v = ptx::ld_shared_v4(slab + r * 128 + ((chunk ^ (r & 7)) << 4));
          const int g = row0 + r;
          uint16_t* dst;
          if (p.own_mode == OWN_SINGLE || p.nvls) {
            dst = reinterpret_cast<uint16_t*>(p.epi_base[0]) + layout_offset(p.epi_layout, g, col);
          } else if (p.own_mode == OWN_BLOCK) {
            const int o = g / p.rows_per_owner;
            const int lr = g - o * p.rows_per_owner;
            dst = reinterpret_cast<uint16_t*>(p.epi_base[o]) + static_cast<long long>(lr) * p.N + col;
          } else {
            const int lr = g / p.ws;
            const int o = g - lr * p.ws;
            dst = reinterpret_cast<uint16_t*>(p.epi_base[o]) + static_cast<long long>(lr) * p.N + col;
          }
          ptx::st_v4(dst, v);
        }
        __syncwarp();
      }

      // ---- progress: this warp's slab of the tile is written ----
      // (__syncwarp above ordered every lane's stores before this release; the
      // signalling warp acquires it and publishes the tile at system scope, so
      // that no epilogue warp ever waits for a system-scope fence.)
      if (lane == 0) ptx::st_release_cta_shared(&epi_prog[q], static_cast<uint32_t>(it + 1));
    }
  } else if (warp == 3) {
    // ===================== signalling =====================
    // One thread per CTA follows the epilogue warps tile by tile: when all four
    // have stored their slabs it fences at system scope and bumps the arrival
    // counter of the tile's 128-row block on the GPU(s) that own those rows,
    // and keeps the reference-compatible counters.
    const bool wanted = p.flag[0] != nullptr || p.seg_counter != nullptr || p.ticket_counter != nullptr;
    if (lane == 0 && wanted) {
      int it = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride, ++it) {
        const uint32_t need = static_cast<uint32_t>(it + 1);
        uint32_t spins = 0;
        while (true) {
          uint32_t lo = ptx::ld_acquire_cta_shared(&epi_prog[0]);
#pragma unroll
          for (int w = 1; w < 4; ++w) {
            const uint32_t v = ptx::ld_acquire_cta_shared(&epi_prog[w]);
            lo = v < lo ? v : lo;
          }
          if (lo >= need) break;
          if ((++spins & 0xffu) == 0u && (*abort_flag || ptx::globaltimer_ns() > deadline)) {
            ok = false;  // the epilogue gave up (it has reported why) or ran out of time
            break;
          }
          __nanosleep(32);
        }
        if (!ok) break;
        int m_blk, n_blk;
        tile_coords(p, t, m_blk, n_blk);
        const int blk_row0 = m_blk * TILE_M + static_cast<int>(cta_rank) * BM;
        const int flag_blk = blk_row0 / BM;
        if (p.flag[0] != nullptr) {
          ptx::fence_acq_rel_sys();
          if (p.nvls) {
            ptx::multimem_red_relaxed_add(p.mc_flag + flag_blk, 1u);  // lands on every rank
          } else if (p.own_mode == OWN_INTERLEAVE) {
            for (int r = 0; r < p.ws; ++r) ptx::red_relaxed_sys_add(p.flag[r] + flag_blk, 1u);
          } else if (p.own_mode == OWN_BLOCK) {
            ptx::red_relaxed_sys_add(p.flag[blk_row0 / p.rows_per_owner] + flag_blk, 1u);
          } else {
            ptx::red_relaxed_sys_add(p.flag[0] + flag_blk, 1u);
          }
        }
        if (p.seg_counter != nullptr || p.ticket_counter != nullptr) {
          // Reference-compatible bookkeeping.
          const int tile_id = m_blk * p.TN + n_blk;
          const int slot = p.slot_of_tile ? p.slot_of_tile[tile_id] : tile_id;
          if (p.seg_counter != nullptr) {
            // Segment counters gate work on another stream of this GPU: every
            // CTA counts its own part of the tile (a CTA pair adds 2 per tile)
            // once its stores are visible device-wide.
            int seg = 0, acc = 0;
            for (; seg < p.nseg; ++seg) {
              acc += p.cseg[seg];
              if (slot < acc) break;
            }
            ptx::fence_acq_rel_gpu();
            if (seg < p.nseg) atomicAdd(p.seg_counter + seg, 1);
          }
          if (cta_rank == 0 && p.ticket_counter != nullptr) {  // completion order, once per tile
            const int ticket = atomicAdd(p.ticket_counter, 1);
            if (slot >= 0 && slot < num_tiles) p.trace[slot] = ticket;
            else report_error(p, ST_BAD_INDEX, 0x500u, slot, num_tiles);
          }
        }
      }
    }
  }

  int group = 0;  // row group of this warp in the reduce phase
  int wg = 0;     // warp inside the group
  if (warp >= kGemmWarps) {
    // ===================== communication warps =====================
    const int cw = warp - kGemmWarps;
    if (p.ag_push) {
      // All-gather / all-to-all push.  This rank's rows of A go to every
      // rank's gathered A, destination by destination: first its own copy (the
      // GEMM starts there), then rank me-1 (which works on this shard right
      // after its own), me-2, ...  Every communication warp of every CTA takes
      // an interleaved share; when a destination's share is written the warp
      // fences at system scope and bumps that rank's shard counter.
      const long long stride = static_cast<long long>(gridDim.x) * (kCommWarps * 32);
      const long long first = static_cast<long long>(blockIdx.x) * (kCommWarps * 32) + cw * 32 + lane;
      if (p.ag_mc_dst != nullptr) {
        // all-gather through the switch: one multicast store per chunk lands on every rank
        const long long chunks = p.ag_bytes[p.me] >> 4;
        const char* src = static_cast<const char*>(p.ag_src[p.me]);
        char* dst = static_cast<char*>(p.ag_mc_dst);
        long long c = first;
        for (; c + 7 * stride < chunks; c += 8 * stride) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint4*>(src + ((c + u * stride) << 4));
#pragma unroll
          for (int u = 0; u < 8; ++u) ptx::multimem_st_v4(dst + ((c + u * stride) << 4), v[u]);
        }
        for (; c < chunks; c += stride) {
          ptx::multimem_st_v4(dst + (c << 4), *reinterpret_cast<const uint4*>(src + (c << 4)));
        }
        __syncwarp();
        if (lane == 0) {
          ptx::fence_acq_rel_sys();
          ptx::multimem_red_relaxed_add(p.ag_mc_flag, 1u);
        }
        return;
      }
      for (int j = 0; j < p.ws; ++j) {
        int d = p.me - j;
        if (d < 0) d += p.ws;
        const long long chunks = p.ag_bytes[d] >> 4;
        const char* src = static_cast<const char*>(p.ag_src[d]);
        char* dst = static_cast<char*>(p.ag_dst[d]);
        long long c = first;
        for (; c + 7 * stride < chunks; c += 8 * stride) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint4*>(src + ((c + u * stride) << 4));
#pragma unroll
          for (int u = 0; u < 8; ++u) ptx::st_v4(dst + ((c + u * stride) << 4), v[u]);
        }
        for (; c < chunks; c += stride) {
          ptx::st_v4(dst + (c << 4), *reinterpret_cast<const uint4*>(src + (c << 4)));
        }
        __syncwarp();
        if (lane == 0) {
          ptx::fence_acq_rel_sys();
          ptx::red_relaxed_sys_add(p.ag_flag[d], 1u);
        }
      }
      if (p.phase_trace != nullptr && lane == 0) {  // when this CTA's share of the push was out
        atomicMax(p.phase_trace + static_cast<unsigned long long>(kTraceWords) * blockIdx.x + 2, ptx::globaltimer_ns());
      }
      return;
    }
    if (!p.reduce) return;
    static_assert(kCommWarps == kGroupWarps, "the communication warps form one row group");
    group = 0;  // reduces rows from the first cycle on
    wg = cw;
  } else {
    // ===================== teardown of the GEMM phase (GEMM warps only) =====================
    __syncwarp();
    ptx::tc_fence_before_sync();
    ptx::named_barrier_sync(8, kGemmThreads);
    if constexpr (CTAS == 2) {
      // The partner may still read this CTA's operands or signal its barriers:
      // each CTA tells the other that its GEMM warps are done and waits (bounded)
      // to hear the same.
      if (threadIdx.x == 0) {
        ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(pair_bar), cta_rank ^ 1u));
        if (!ptx::mbar_wait_cluster(pair_bar, 0u, deadline)) {
          report_error(p, ST_TIMEOUT_PIPE, 0x700u, 0, 0);
          *abort_flag = 1;
        }
      }
      ptx::named_barrier_sync(8, kGemmThreads);
    }
    if (warp == 2) {
      ptx::tc_fence_after_sync();
      if constexpr (CTAS == 2) ptx::tmem_dealloc_pair(tmem_base, T::TMEM_COLS);
      else ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
    }
    if (p.phase_trace != nullptr && threadIdx.x == 0) {
      unsigned long long* tr = p.phase_trace + static_cast<unsigned long long>(kTraceWords) * blockIdx.x;
      tr[1] = ptx::globaltimer_ns();
      int mine = 0;
      for (int t = first_tile; t < num_tiles; t += tile_stride) ++mine;
      tr[3] = static_cast<unsigned long long>(mine);
    }
    if (!p.reduce || *abort_flag) return;
    // out of tiles: the GEMM warps join the reduce phase as two more row groups
    group = 1 + warp / kGroupWarps;  // warps 0-3 -> group 1, warps 4-7 -> group 2
    wg = warp % kGroupWarps;
  }

  // ===================== reduce phase (every warp ends up here) =====================
  comm_dispatch<BF16>(p, group_scratch + group, gamma_smem, group, wg, lane, deadline, abort_flag);

  // All-reduce: the kernel may only end once every owner has delivered its
  // rows into this rank's output.
  if (p.bcast && blockIdx.x == 0 && threadIdx.x == 0 && p.done[p.me] != nullptr) {
    uint32_t seen = 0;
    if (!ptx::wait_counter_geq(p.done[p.me], p.done_target, deadline, &seen)) {
      report_error(p, ST_TIMEOUT_DONE, 0, seen, p.done_target);
    }
    if (p.phase_trace != nullptr) p.phase_trace[6] = ptx::globaltimer_ns();
  }
}

}  // namespace fo
