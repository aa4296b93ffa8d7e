// Persistent, warp-specialised sm_100a kernel: C = A * B^T on tcgen05 tensor
// cores with TMEM accumulators, operands staged by TMA, and the collective that
// follows the GEMM (all-reduce or reduce-scatter, optionally RMSNorm) fused in
// through peer-to-peer stores and system-scope counters.
//
// CTA layout (256 threads, one CTA per SM, grid <= number of SMs):
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads; with a
//                               gathered A operand it first waits for the source
//                               ranks whose rows the tile needs)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma / tcgen05.commit)
//   warp 2      TMEM allocator (allocates 2 x BN columns, frees them at the end);
//                               in all-gather / all-to-all mode it then pushes this
//                               rank's rows of A to the other ranks
//   warp 3      signalling     (one lane publishes finished tiles at system scope
//                               and bumps the owners' arrival counters)
//   warps 4-7   epilogue       (tcgen05.ld -> convert -> smem transpose ->
//                               coalesced 16-byte stores, local or to a peer)
// With CTAS == 2 two such CTAs form a cluster: both stage operands and run an
// epilogue for their own 128 rows, the MMA warp of rank 0 issues for the pair.
// After its last tile the whole CTA joins the reduce phase: groups of 1, 2, 4 or
// 8 warps take one owned row at a time.
//
// Replaces, as one launch, the reference's signalling GEMM + wait kernel +
// segmented NCCL calls (reference: src/overlap_impl.cu:221-328).
#pragma once

#include "fused_params.h"
#include "sm100_ptx.cuh"

namespace fo {

// CTAS == 1: one CTA computes a 128 x BN tile (tcgen05.mma.cta_group::1).
// CTAS == 2: a cluster of two CTAs computes a 256 x BN tile with
//   tcgen05.mma.cta_group::2; each CTA stages its own 128 rows of A and one
//   half of the B tile, so every SM fetches a third less per FLOP.
template <int BN_, int CTAS_ = 1>
struct TileTraits {
  static constexpr int CTAS = CTAS_;
  static constexpr int BM = 128;           // rows per CTA
  static constexpr int TILE_M = BM * CTAS;  // rows per tile
  static constexpr int BN = BN_;
  static constexpr int BK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
  static constexpr int UMMA_K = 16;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_ROWS = BN / CTAS;  // rows of B staged by each CTA
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_WARPS = 4;
  static constexpr int EPI_SLAB_BYTES = 32 * 128;  // 32 rows x 64 columns of 16-bit values
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_SLAB_BYTES;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_LIMIT = 227 * 1024;
  static constexpr int STAGES_RAW = (SMEM_LIMIT - 1024 - EPI_BYTES - BAR_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulator buffers; power of two >= 32
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
  static_assert(CTAS == 1 || CTAS == 2, "one CTA or a CTA pair");
  static_assert(STAGES >= 3, "pipeline too shallow");
};

constexpr int kThreads = 256;

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

__device__ __forceinline__ void report_error(StatusWord* st, uint32_t code, uint32_t rank, uint32_t where,
                                             uint32_t seen, uint32_t want) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->rank = rank;
    st->where = where;
    st->seen = seen;
    st->want = want;
    __threadfence_system();
  }
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

// Tile order: tile rows are walked in groups of `raster_group`; inside a group
// the walk is column-major so that one B panel serves the whole group from L2
// and tile rows still complete early and in order.
__device__ __forceinline__ void tile_coords(const FusedParams& p, int t, int& m_blk, int& n_blk) {
  const int G = p.raster_group;
  const int per_group = G * p.TN;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int first = g * G;
  const int rows_here = (p.TM - first) < G ? (p.TM - first) : G;
  const int mb = first + r % rows_here;
  n_blk = r / rows_here;
  m_blk = mb + p.rot;
  if (m_blk >= p.TM) m_blk -= p.TM;
}

// ---------------------------------------------------------------------------
// reduce phase: a group of G warps per owned row (G = p.reduce_group)
// ---------------------------------------------------------------------------
// Each group takes one row at a time: its warps wait (bounded) until the
// partial rows of every rank have arrived, sum them in fp32 and round the sum
// to the 16-bit type (the value an all-reduce would have produced).  Without
// RMSNorm the rounded sum goes straight to its destination(s); with RMSNorm it
// is parked in shared memory while the sum of squares is accumulated (combined
// across the group's warps through a named barrier when G > 1), then scaled,
// multiplied by the weight and written out.  Groups never synchronise with one
// another, so every SM keeps several independent chains of loads in flight.
// NVLS == true replaces the per-rank loads by one multimem.ld_reduce per chunk
// and the per-rank result stores by one multimem.st.  WS > 0 fixes the number of ranks at compile time (all
// loads of a batch are issued before the first use); WS == 0 is the generic
// fallback for other group sizes.
template <bool BF16, int WS, bool NVLS>
__device__ __forceinline__ void reduce_phase(const FusedParams& p, uint8_t* smem, int smem_bytes, float* red,
                                             int warp, int lane, uint64_t deadline, volatile uint32_t* abort_flag) {
  constexpr int BM = 128;
  // NVLS: one load-reduce per chunk replaces the ws loads (instantiated with WS == 1)
  constexpr int U = WS == 0 ? 1 : (WS == 1 ? 8 : (WS == 2 ? 4 : 2));  // chunks per lane per batch
  constexpr int NS = WS == 0 ? kMaxRanks : WS;
  constexpr int kWarps = kThreads / 32;
  const int ws = NVLS ? p.ws : (WS == 0 ? p.ws : WS);
  const int nsrc = NVLS ? 1 : ws;  // loads per chunk
  const int n_chunks = p.N >> 3;  // 16-byte chunks per row
  const int row_bytes = p.N * 2;
  const uint32_t smem_base = ptx::smem_u32(smem);
  // G warps share one row (G = 1, 2, 4 or 8); few rows per CTA -> larger G
  const int G = p.reduce_group;
  int groups = kWarps / G;
  const int gidx = warp / G;  // row group of this warp
  const int wg = warp - gidx * G;

  // RMSNorm: the weight vector is staged in shared memory once per CTA, then
  // one row buffer per row group follows it.
  if (p.norm) {
    const uint16_t* gamma = reinterpret_cast<const uint16_t*>(p.gamma);
    for (int c = threadIdx.x; c < n_chunks; c += kThreads) {
      ptx::st_shared_v4(smem_base + (static_cast<uint32_t>(c) << 4), *reinterpret_cast<const uint4*>(gamma + c * 8));
    }
    const int fit = (smem_bytes - row_bytes) / row_bytes;
    if (fit < groups) groups = fit;
    __syncthreads();
  }
  if (groups < 1 || gidx >= groups) return;  // (< 1 is rejected on the host)
  const uint32_t gbuf = smem_base;
  const uint32_t rowbuf = smem_base + static_cast<uint32_t>(row_bytes) * static_cast<uint32_t>(gidx + 1);
  const int rows_local = p.rows_per_owner;
  const uint16_t* stage = reinterpret_cast<const uint16_t*>(p.stage);
  const long long src_stride = static_cast<long long>(rows_local) * p.N;
  const uint32_t* my_flag = p.flag[p.me];
  const int cl = wg * 32 + lane;  // first chunk of this lane
  const int cstep = 32 * G;       // chunk stride between a lane's chunks

  auto load_batch = [&](uint4 (&v)[U][NS], const uint16_t* src0, int c0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + cstep * u;
      if (c < n_chunks) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          if (s < nsrc) {
            if constexpr (NVLS) v[u][s] = ptx::multimem_ld_reduce_add_v4<BF16>(src0 + c * 8);
            else v[u][s] = ptx::ld_cg_v4(src0 + s * src_stride + c * 8);
          }
        }
      }
    }
  };
  auto store_out = [&](int out_row, int c, const uint4& o) {
    const long long off = layout_offset(p.out_layout, out_row, c * 8);
    if (NVLS && p.bcast) {
      ptx::multimem_st_v4(reinterpret_cast<uint16_t*>(p.mc_out) + off, o);  // lands on every rank
    } else if (p.bcast) {
#pragma unroll
      for (int r = 0; r < NS; ++r) {
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

  for (int i = 0;; ++i) {
    const int lr = static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) * (gidx + groups * i);
    if (lr >= rows_local) break;
    int g;  // global row
    if (p.own_mode == OWN_BLOCK) g = p.me * rows_local + lr;
    else if (p.own_mode == OWN_INTERLEAVE) g = lr * ws + p.me;
    else g = lr;
    const int rb = g / BM;

    // wait until every rank's partials for tile row rb have arrived
    uint32_t ok = 1;
    if (lane == 0) {
      uint32_t seen = 0;
      if (!ptx::wait_counter_geq(my_flag + rb, p.flag_target, deadline, &seen)) {
        report_error(p.status, ST_TIMEOUT_FLAG, p.me, rb, seen, p.flag_target);
        *abort_flag = 1;
        ok = 0;
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);

    const int out_row = p.bcast ? g : lr;
    // NVLS: partials sit at their global row in every rank's staging buffer
    const uint16_t* src0 = NVLS ? reinterpret_cast<const uint16_t*>(p.mc_stage) + static_cast<long long>(g) * p.N
                                : stage + static_cast<long long>(lr) * p.N;
    float ssq = 0.f;
    if (ok) {
      // software pipeline: the loads of batch k+1 are in flight while batch k is summed
      uint4 cur[U][NS], nxt[U][NS];
      load_batch(cur, src0, cl);
      for (int c0 = cl; c0 < n_chunks; c0 += cstep * U) {
        if (c0 + cstep * U < n_chunks) load_batch(nxt, src0, c0 + cstep * U);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + cstep * u;
          if (c < n_chunks) {
            float a[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = 0.f;
#pragma unroll
            for (int s = 0; s < NS; ++s) {
              if (s < nsrc) {
                float2 f;
                f = unpack2<BF16>(cur[u][s].x); a[0] += f.x; a[1] += f.y;
                f = unpack2<BF16>(cur[u][s].y); a[2] += f.x; a[3] += f.y;
                f = unpack2<BF16>(cur[u][s].z); a[4] += f.x; a[5] += f.y;
                f = unpack2<BF16>(cur[u][s].w); a[6] += f.x; a[7] += f.y;
              }
            }
            uint4 h;
            h.x = pack2<BF16>(a[0], a[1]);
            h.y = pack2<BF16>(a[2], a[3]);
            h.z = pack2<BF16>(a[4], a[5]);
            h.w = pack2<BF16>(a[6], a[7]);
            if (p.norm) {
              float2 f;
              f = unpack2<BF16>(h.x); ssq += f.x * f.x + f.y * f.y;
              f = unpack2<BF16>(h.y); ssq += f.x * f.x + f.y * f.y;
              f = unpack2<BF16>(h.z); ssq += f.x * f.x + f.y * f.y;
              f = unpack2<BF16>(h.w); ssq += f.x * f.x + f.y * f.y;
              ptx::st_shared_v4(rowbuf + (static_cast<uint32_t>(c) << 4), h);
            } else {
              store_out(out_row, c, h);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int s = 0; s < NS; ++s) cur[u][s] = nxt[u][s];
        }
      }
    }
    if (p.norm) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if (G > 1) {
        // combine the partial sums of the G warps of this row group; the slot
        // alternates with the row so that a fast warp cannot overwrite a value
        // a slow warp of the same group has yet to read
        float* slot = red + (i & 1) * kWarps + gidx * G;
        if (lane == 0) slot[wg] = ssq;
        asm volatile("bar.sync %0, %1;" ::"r"(1 + gidx), "r"(G * 32) : "memory");
        ssq = 0.f;
        for (int w = 0; w < G; ++w) ssq += slot[w];
      }
      if (ok) {
        const float rstd = rsqrtf(ssq / static_cast<float>(p.N) + p.eps);
        // each lane re-reads exactly the chunks it wrote, so no barrier is needed for the row buffer
#pragma unroll 4
        for (int c = cl; c < n_chunks; c += cstep) {
          const uint4 h = ptx::ld_shared_v4(rowbuf + (static_cast<uint32_t>(c) << 4));
          const uint4 w = ptx::ld_shared_v4(gbuf + (static_cast<uint32_t>(c) << 4));
          float2 f;
          uint4 o;
          f = unpack2<BF16>(h.x); o.x = norm_pack2<BF16>(f.x, f.y, rstd, w.x);
          f = unpack2<BF16>(h.y); o.y = norm_pack2<BF16>(f.x, f.y, rstd, w.y);
          f = unpack2<BF16>(h.z); o.z = norm_pack2<BF16>(f.x, f.y, rstd, w.z);
          f = unpack2<BF16>(h.w); o.w = norm_pack2<BF16>(f.x, f.y, rstd, w.w);
          store_out(out_row, c, o);
        }
      }
    }
    if (!ok) continue;  // keep taking part in the group barriers of later rows; their waits fail at once
    if (p.bcast) {
      __syncwarp();  // every lane's stores of this row part precede the releases below
      if constexpr (NVLS) {
        if (lane == 0) ptx::multimem_red_release_add(p.mc_done, 1u);
      } else {
        if (lane < ws && p.done[lane] != nullptr) ptx::red_release_sys_add(p.done[lane], 1u);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// reduce phase on a single GPU with RMSNorm: rows streamed through shared memory
// ---------------------------------------------------------------------------
// With one rank there is nothing to sum: the phase is RMSNorm over the product
// the epilogue stored.  Eight warps per SM cannot hide memory latency with
// register loads, so each warp keeps two row buffers in shared memory and lets
// the bulk-copy engine fetch row i+1 (cp.async.bulk, completion on an mbarrier)
// while it normalises row i out of shared memory.  Returns false without doing
// anything when shared memory cannot hold two rows per warp for at least one
// warp (the caller then takes the generic path).
template <bool BF16>
__device__ __forceinline__ bool reduce_phase_single(const FusedParams& p, uint8_t* smem, int smem_bytes,
                                                    uint64_t* rbar, int warp, int lane, uint64_t deadline,
                                                    volatile uint32_t* abort_flag) {
  constexpr int BM = 128;
  constexpr int kWarps = kThreads / 32;
  const int n_chunks = p.N >> 3;
  const int row_bytes = p.N * 2;
  int active = ((smem_bytes - row_bytes) / row_bytes) / 2;  // warps that get two row buffers after the weight vector
  if (active > kWarps) active = kWarps;
  if (active < 1) return false;
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint16_t* gamma = reinterpret_cast<const uint16_t*>(p.gamma);
  for (int c = threadIdx.x; c < n_chunks; c += kThreads) {
    ptx::st_shared_v4(smem_base + (static_cast<uint32_t>(c) << 4), *reinterpret_cast<const uint4*>(gamma + c * 8));
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * kWarps; ++i) ptx::mbar_init(&rbar[i], 1);
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp >= active) return true;
  const uint32_t buf0 = smem_base + static_cast<uint32_t>(row_bytes) * static_cast<uint32_t>(1 + 2 * warp);
  uint64_t* bar = rbar + 2 * warp;
  const int rows_local = p.rows_per_owner;
  const uint16_t* stage = reinterpret_cast<const uint16_t*>(p.stage);
  const uint32_t* my_flag = p.flag[p.me];
  auto row_of = [&](int i) { return static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) * (warp + active * i); };

  // lane 0: wait for the row's tile row, then start the copy of row i into buffer b
  auto issue = [&](int i, int b) -> uint32_t {
    const int lr = row_of(i);
    if (lr >= rows_local) return 1u;
    const int rb = lr / BM;
    uint32_t seen = 0;
    if (!ptx::wait_counter_geq(my_flag + rb, p.flag_target, deadline, &seen)) {
      report_error(p.status, ST_TIMEOUT_FLAG, p.me, rb, seen, p.flag_target);
      *abort_flag = 1;
      return 0u;
    }
    ptx::fence_proxy_async_all();  // the epilogue's generic-proxy stores before the async-proxy read
    ptx::mbar_arrive_expect_tx(&bar[b], static_cast<uint32_t>(row_bytes));
    ptx::bulk_load_1d(buf0 + static_cast<uint32_t>(b * row_bytes), stage + static_cast<long long>(lr) * p.N,
                      static_cast<uint32_t>(row_bytes), &bar[b]);
    return 1u;
  };

  uint32_t ok = 1;
  if (lane == 0) ok = issue(0, 0);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  uint32_t phases = 0;  // bit b: parity to wait for on buffer b
  for (int i = 0; ok; ++i) {
    const int lr = row_of(i);
    if (lr >= rows_local) break;
    const int b = i & 1;
    // all lanes finished reading buffer b^1 (row i-1) at the __syncwarp below
    if (lane == 0) ok = issue(i + 1, b ^ 1);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ptx::mbar_wait(&bar[b], (phases >> b) & 1u, deadline)) {
      if (lane == 0) {
        report_error(p.status, ST_TIMEOUT_PIPE, p.me, 0x600u + warp, i, lr);
        *abort_flag = 1;
      }
      break;
    }
    phases ^= 1u << b;
    const uint32_t rowbuf = buf0 + static_cast<uint32_t>(b * row_bytes);
    float ssq = 0.f;
#pragma unroll 4
    for (int c = lane; c < n_chunks; c += 32) {
      const uint4 h = ptx::ld_shared_v4(rowbuf + (static_cast<uint32_t>(c) << 4));
      float2 f;
      f = unpack2<BF16>(h.x); ssq += f.x * f.x + f.y * f.y;
      f = unpack2<BF16>(h.y); ssq += f.x * f.x + f.y * f.y;
      f = unpack2<BF16>(h.z); ssq += f.x * f.x + f.y * f.y;
      f = unpack2<BF16>(h.w); ssq += f.x * f.x + f.y * f.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    const float rstd = rsqrtf(ssq / static_cast<float>(p.N) + p.eps);
#pragma unroll 4
    for (int c = lane; c < n_chunks; c += 32) {
      const uint4 h = ptx::ld_shared_v4(rowbuf + (static_cast<uint32_t>(c) << 4));
      const uint4 w = ptx::ld_shared_v4(smem_base + (static_cast<uint32_t>(c) << 4));
      float2 f;
      uint4 o;
      f = unpack2<BF16>(h.x); o.x = norm_pack2<BF16>(f.x, f.y, rstd, w.x);
      f = unpack2<BF16>(h.y); o.y = norm_pack2<BF16>(f.x, f.y, rstd, w.y);
      f = unpack2<BF16>(h.z); o.z = norm_pack2<BF16>(f.x, f.y, rstd, w.z);
      f = unpack2<BF16>(h.w); o.w = norm_pack2<BF16>(f.x, f.y, rstd, w.w);
      ptx::st_v4(reinterpret_cast<uint16_t*>(p.out[0]) + layout_offset(p.out_layout, lr, c * 8), o);
    }
    __syncwarp();
    if (p.bcast && lane == 0 && p.done[0] != nullptr) ptx::red_release_sys_add(p.done[0], 1u);
  }
  return true;
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int BN, bool BF16, int CTAS>
__global__ void __launch_bounds__(kThreads, 1) gemm_fused_sm100_kernel(const __grid_constant__ FusedParams p) {
  using T = TileTraits<BN, CTAS>;
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
  uint64_t* full_bar = bars;                   // [STAGES] TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;         // [STAGES] MMA -> TMA
  uint64_t* tfull_bar = bars + 2 * STAGES;     // [2] MMA -> epilogue
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* epi_prog = tmem_slot + 4;  // [4] tiles finished by each epilogue warp
  float* red = reinterpret_cast<float*>(bars + 40);  // [2][8] partial sums of the reduce phase

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
    *abort_flag = 0;
    for (int i = 0; i < 4; ++i) epi_prog[i] = 0;
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&p.tmA);
    ptx::prefetch_tensormap(&p.tmB);
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
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
        int m_blk, n_blk;
        tile_coords(p, t, m_blk, n_blk);
        const int a_row = m_blk * TILE_M + static_cast<int>(cta_rank) * BM;
        const int b_row = n_blk * BN + static_cast<int>(cta_rank) * T::B_ROWS;
        if (p.a_ready != nullptr) {
          // Gathered A: wait until every source rank whose rows overlap
          // [a_row, a_row + BM) has delivered them into local memory, then order
          // those generic-proxy writes before the async-proxy (TMA) reads.
          for (int r = 0; r < p.ws && ok; ++r) {
            const int r_begin = r == 0 ? 0 : p.a_src_end[r - 1];
            const int r_end = p.a_src_end[r];
            if (r_end <= r_begin || r_end <= a_row || r_begin >= a_row + BM) continue;
            uint32_t seen = 0;
            if (!ptx::wait_counter_geq(p.a_ready + r, p.a_ready_target, deadline, &seen)) {
              report_error(p.status, ST_TIMEOUT_GATHER, p.me, r, seen, p.a_ready_target);
              *abort_flag = 1;
              ok = false;
            }
          }
          if (!ok) break;
          ptx::fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, deadline)) {
            report_error(p.status, ST_TIMEOUT_PIPE, p.me, 0x100u + stage, kb, t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if constexpr (CTAS == 2) {
            // both CTAs' bytes are counted on the leader's barrier
            if (cta_rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * T::STAGE_BYTES);
            ptx::tma_load_2d_pair(smem_a + stage * T::A_BYTES, &p.tmA, &full_bar[stage], kb * BK, a_row);
            ptx::tma_load_2d_pair(smem_b + stage * T::B_BYTES, &p.tmB, &full_bar[stage], kb * BK, b_row);
          } else {
            ptx::mbar_arrive_expect_tx(&full_bar[stage], T::STAGE_BYTES);
            ptx::tma_load_2d(smem_a + stage * T::A_BYTES, &p.tmA, &full_bar[stage], kb * BK, a_row);
            ptx::tma_load_2d(smem_b + stage * T::B_BYTES, &p.tmB, &full_bar[stage], kb * BK, b_row);
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
            report_error(p.status, ST_TIMEOUT_GATHER, p.me, 0x100u + r, seen, p.a_ready_target);
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
          report_error(p.status, ST_TIMEOUT_PIPE, p.me, 0x200u + buf, it, t);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, deadline)) {
            report_error(p.status, ST_TIMEOUT_PIPE, p.me, 0x300u + stage, kb, t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint64_t da = ptx::make_smem_desc_k_sw128(ptx::smem_u32(smem_a + stage * T::A_BYTES));
          const uint64_t db = ptx::make_smem_desc_k_sw128(ptx::smem_u32(smem_b + stage * T::B_BYTES));
#pragma unroll
          for (int k = 0; k < BK / T::UMMA_K; ++k) {
            // advancing K by 16 elements = 32 bytes = 2 descriptor address units
            if constexpr (CTAS == 2) ptx::umma_f16_ss_pair(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else ptx::umma_f16_ss(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
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
  } else if (warp == 2) {
    // ===================== all-gather push =====================
    // This rank's shard of A goes to every rank's gathered A, destination by
    // destination: first its own copy (the GEMM starts there), then rank me-1
    // (which works on this shard right after its own), me-2, ...  Warp 2 of every CTA takes an
    // interleaved share; when a destination's share is written the warp fences
    // at system scope and bumps that rank's shard counter.
    if (p.ag_push) {
      const long long stride = static_cast<long long>(gridDim.x) * 32;
      const long long first = static_cast<long long>(blockIdx.x) * 32 + lane;
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
    }
  } else if (warp >= 4) {
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
          report_error(p.status, ST_TIMEOUT_PIPE, p.me, 0x400u + buf, it, t);
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
            else report_error(p.status, ST_BAD_INDEX, p.me, 0x500u, slot, num_tiles);
          }
        }
      }
    }
  }

  // ===================== teardown of the GEMM phase =====================
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (CTAS == 2) ptx::cluster_sync();  // the partner may still read this CTA's operands / signal its barriers
  if (warp == 2) {
    ptx::tc_fence_after_sync();
    if constexpr (CTAS == 2) ptx::tmem_dealloc_pair(tmem_base, T::TMEM_COLS);
    else ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
  if (p.phase_trace != nullptr && threadIdx.x == 0) {
    unsigned long long* tr = p.phase_trace + 4ull * blockIdx.x;
    tr[0] = t_start;
    tr[1] = ptx::globaltimer_ns();
    tr[2] = 0;
    int mine = 0;
    for (int t = first_tile; t < num_tiles; t += tile_stride) ++mine;
    tr[3] = static_cast<unsigned long long>(mine);
  }
  if (!p.reduce || *abort_flag) return;

  // ===================== reduce phase =====================
  ptx::fence_proxy_async_smem();  // the pipeline's shared memory is reused through the generic proxy
  constexpr int kRowSmem = T::STAGES * T::STAGE_BYTES + T::EPI_BYTES;
  // barriers of the single-GPU row pipeline: behind the partial-sum scratch
  uint64_t* rbar = bars + 48;
  if (p.nvls) {
    reduce_phase<BF16, 1, true>(p, smem, kRowSmem, red, warp, lane, deadline, abort_flag);
  } else if (p.ws == 1 && p.norm && p.reduce_group == 1 &&
             reduce_phase_single<BF16>(p, smem, kRowSmem, rbar, warp, lane, deadline, abort_flag)) {
    // done: rows streamed through shared memory
  } else {
    switch (p.ws) {
      case 1: reduce_phase<BF16, 1, false>(p, smem, kRowSmem, red, warp, lane, deadline, abort_flag); break;
      case 2: reduce_phase<BF16, 2, false>(p, smem, kRowSmem, red, warp, lane, deadline, abort_flag); break;
      case 4: reduce_phase<BF16, 4, false>(p, smem, kRowSmem, red, warp, lane, deadline, abort_flag); break;
      case 8: reduce_phase<BF16, 8, false>(p, smem, kRowSmem, red, warp, lane, deadline, abort_flag); break;
      default: reduce_phase<BF16, 0, false>(p, smem, kRowSmem, red, warp, lane, deadline, abort_flag); break;
    }
  }

  if (p.phase_trace != nullptr && lane == 0) {
    atomicMax(p.phase_trace + 4ull * blockIdx.x + 2, static_cast<unsigned long long>(ptx::globaltimer_ns()));
  }

  // All-reduce: the kernel may only end once every owner has delivered its
  // rows into this rank's output.
  if (p.bcast && blockIdx.x == 0 && threadIdx.x == 0 && p.done[p.me] != nullptr) {
    uint32_t seen = 0;
    if (!ptx::wait_counter_geq(p.done[p.me], p.done_target, deadline, &seen)) {
      report_error(p.status, ST_TIMEOUT_DONE, p.me, 0, seen, p.done_target);
    }
  }
}

}  // namespace fo
