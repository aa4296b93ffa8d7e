// Persistent, warp-specialised sm_100a kernel: C = A * B^T on tcgen05 tensor
// cores with TMEM accumulators, operands staged by TMA, and the collective that
// follows the GEMM (all-reduce or reduce-scatter, optionally RMSNorm) fused in
// through peer-to-peer stores and system-scope counters.
//
// CTA layout (256 threads, one CTA per SM, grid <= number of SMs):
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma / tcgen05.commit)
//   warp 2      TMEM allocator (allocates 2 x BN columns, frees them at the end)
//   warp 3      idle during the GEMM phase
//   warps 4-7   epilogue       (tcgen05.ld -> convert -> smem transpose ->
//                               coalesced 16-byte stores -> arrival counter)
// After its last tile the whole CTA joins the reduce phase (row-per-CTA).
//
// Replaces, as one launch, the reference's signalling GEMM + wait kernel +
// segmented NCCL calls (reference: src/overlap_impl.cu:221-328).
#pragma once

#include "fused_params.h"
#include "sm100_ptx.cuh"

namespace fo {

template <int BN_>
struct TileTraits {
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr int BK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
  static constexpr int UMMA_K = 16;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
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
  static_assert(STAGES >= 3, "pipeline too shallow");
};

constexpr int kThreads = 256;
constexpr int kMaxRowChunksPerThread = 8;  // reduce phase: N <= 8 * 256 * 8 = 16384

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ long long layout_offset(const OutLayout& L, int row, int col) {
  if (!L.tiled) return static_cast<long long>(row) * L.ld + col;
  const int t = (row / L.bm) * L.tn + col / L.bn;
  const int s = L.ra ? L.ra[t] : t;
  const long long w = static_cast<long long>(L.rldn) * L.bn;
  return (static_cast<long long>(s / L.rldn) * L.bm + row % L.bm) * w + (s % L.rldn) * L.bn + col % L.bn;
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
// the kernel
// ---------------------------------------------------------------------------
template <int BN, bool BF16>
__global__ void __launch_bounds__(kThreads, 1) gemm_fused_sm100_kernel(const __grid_constant__ FusedParams p) {
  using T = TileTraits<BN>;
  constexpr int BM = T::BM, BK = T::BK, STAGES = T::STAGES;

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
  float* red_buf = reinterpret_cast<float*>(tmem_slot + 2);  // [8] block-reduce scratch

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t deadline = ptx::globaltimer_ns() + p.timeout_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], T::EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&p.tmA);
    ptx::prefetch_tensormap(&p.tmB);
  }
  if (warp == 2) {
    ptx::tmem_alloc(tmem_slot, T::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(p, t, m_blk, n_blk);
        if (p.a_ready != nullptr) {
          // All-gathered A: rows of this tile come from one source rank; wait
          // until that shard has landed in local memory, then order the
          // generic-proxy arrival before the async-proxy (TMA) reads.
          const int src = (m_blk * BM) / p.a_rows_per_rank;
          uint32_t seen = 0;
          if (!ptx::wait_counter_geq(p.a_ready + src, p.a_ready_target, deadline, &seen)) {
            report_error(p.status, ST_TIMEOUT_GATHER, p.me, src, seen, p.a_ready_target);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, deadline)) {
            report_error(p.status, ST_TIMEOUT_PIPE, p.me, 0x100u + stage, kb, t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&full_bar[stage], T::STAGE_BYTES);
          ptx::tma_load_2d(smem_a + stage * T::A_BYTES, &p.tmA, &full_bar[stage], kb * BK, m_blk * BM);
          ptx::tma_load_2d(smem_b + stage * T::B_BYTES, &p.tmB, &full_bar[stage], kb * BK, n_blk * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
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
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(BF16 ? 1 : 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
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
            ptx::umma_f16_ss(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[stage]);  // frees the stage once the MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit(&tfull_bar[buf]);  // accumulator complete
      }
    }
  } else if (warp >= 4) {
    // ===================== epilogue =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t slab = ptx::smem_u32(smem_epi + q * T::EPI_SLAB_BYTES);
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
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
      const int row0 = m_blk * BM + q * 32;  // first global row of this warp's slab

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
          if (lane == 0) ptx::mbar_arrive(&tempty_bar[buf]);
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
          if (p.own_mode == OWN_SINGLE) {
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

      // ---- signalling: the slab is written; make it visible, then count ----
      if (p.flag[0] != nullptr) {
        // __syncwarp above ordered every lane's stores before this point; the
        // release on the reduction publishes them at system scope.
        if (p.own_mode == OWN_INTERLEAVE) {
          if (lane < p.ws) ptx::red_release_sys_add(p.flag[lane] + m_blk, 1u);
        } else if (p.own_mode == OWN_BLOCK) {
          if (lane == 0) ptx::red_release_sys_add(p.flag[row0 / p.rows_per_owner] + m_blk, 1u);
        } else {
          if (lane == 0) ptx::red_release_sys_add(p.flag[0] + m_blk, 1u);
        }
      }
      if (q == 0 && lane == 0 && (p.seg_counter != nullptr || p.ticket_counter != nullptr)) {
        // Reference-compatible bookkeeping, once per tile.  (The three other
        // epilogue warps of this tile may still be storing; consumers of these
        // counters run after the kernel, in stream order.)
        const int tile_id = m_blk * p.TN + n_blk;
        const int slot = p.slot_of_tile ? p.slot_of_tile[tile_id] : tile_id;
        if (p.seg_counter != nullptr) {
          int seg = 0, acc = 0;
          for (; seg < p.nseg; ++seg) {
            acc += p.cseg[seg];
            if (slot < acc) break;
          }
          if (seg < p.nseg) atomicAdd(p.seg_counter + seg, 1);
        }
        if (p.ticket_counter != nullptr) {
          const int ticket = atomicAdd(p.ticket_counter, 1);
          if (slot >= 0 && slot < num_tiles) p.trace[slot] = ticket;
          else report_error(p.status, ST_BAD_INDEX, p.me, 0x500u, slot, num_tiles);
        }
      }
    }
  }

  // ===================== teardown of the GEMM phase =====================
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
  if (!p.reduce || *abort_flag) return;

  // ===================== reduce phase =====================
  // One CTA per owned row: sum the ws partial rows in fp32, optionally
  // RMS-normalise, write the row to its destination(s).
  const int n_chunks = p.N / 8;  // 16-byte chunks per row
  const int rows_local = p.rows_per_owner;
  const uint16_t* stage = reinterpret_cast<const uint16_t*>(p.stage);
  const long long src_stride = static_cast<long long>(rows_local) * p.N;
  const uint32_t* my_flag = p.flag[p.me];

  for (int lr = blockIdx.x; lr < rows_local; lr += gridDim.x) {
    int g;  // global row
    if (p.own_mode == OWN_BLOCK) g = p.me * rows_local + lr;
    else if (p.own_mode == OWN_INTERLEAVE) g = lr * p.ws + p.me;
    else g = lr;
    const int rb = g / BM;

    // wait until every rank's partials for tile row rb have arrived
    if (threadIdx.x == 0) {
      uint32_t seen = 0;
      if (!ptx::wait_counter_geq(my_flag + rb, p.flag_target, deadline, &seen)) {
        report_error(p.status, ST_TIMEOUT_FLAG, p.me, rb, seen, p.flag_target);
        *abort_flag = 1;
      }
    }
    __syncthreads();
    if (*abort_flag) return;

    float acc[kMaxRowChunksPerThread][8];
    float ssq = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxRowChunksPerThread; ++k) {
      const int c = threadIdx.x + k * kThreads;
      if (c < n_chunks) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
        const uint16_t* src = stage + static_cast<long long>(lr) * p.N + c * 8;
        uint4 v[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < p.ws) v[s] = ptx::ld_cg_v4(src + s * src_stride);
        }
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < p.ws) {
            float2 f;
            f = unpack2<BF16>(v[s].x); acc[k][0] += f.x; acc[k][1] += f.y;
            f = unpack2<BF16>(v[s].y); acc[k][2] += f.x; acc[k][3] += f.y;
            f = unpack2<BF16>(v[s].z); acc[k][4] += f.x; acc[k][5] += f.y;
            f = unpack2<BF16>(v[s].w); acc[k][6] += f.x; acc[k][7] += f.y;
          }
        }
        if (p.norm) {
#pragma unroll
          for (int e = 0; e < 8; ++e) ssq += acc[k][e] * acc[k][e];
        }
      }
    }
    float rstd = 1.f;
    if (p.norm) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if (lane == 0) red_buf[warp] = ssq;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) tot += red_buf[w];
      rstd = rsqrtf(tot / static_cast<float>(p.N) + p.eps);
    }
    const int out_row = p.bcast ? g : lr;
#pragma unroll
    for (int k = 0; k < kMaxRowChunksPerThread; ++k) {
      const int c = threadIdx.x + k * kThreads;
      if (c < n_chunks) {
        uint4 v;
        if (p.norm) {
          const uint4 w = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.gamma) + c * 8);
          v.x = norm_pack2<BF16>(acc[k][0], acc[k][1], rstd, w.x);
          v.y = norm_pack2<BF16>(acc[k][2], acc[k][3], rstd, w.y);
          v.z = norm_pack2<BF16>(acc[k][4], acc[k][5], rstd, w.z);
          v.w = norm_pack2<BF16>(acc[k][6], acc[k][7], rstd, w.w);
        } else {
          v.x = pack2<BF16>(acc[k][0], acc[k][1]);
          v.y = pack2<BF16>(acc[k][2], acc[k][3]);
          v.z = pack2<BF16>(acc[k][4], acc[k][5]);
          v.w = pack2<BF16>(acc[k][6], acc[k][7]);
        }
        const long long off = layout_offset(p.out_layout, out_row, c * 8);
        if (p.bcast) {
          for (int r = 0; r < p.ws; ++r) {
            // start with the next rank so that the eight owners do not all
            // write to the same destination at the same moment
            int d = p.me + 1 + r;
            if (d >= p.ws) d -= p.ws;
            ptx::st_v4(reinterpret_cast<uint16_t*>(p.out[d]) + off, v);
          }
        } else {
          ptx::st_v4(reinterpret_cast<uint16_t*>(p.out[p.me]) + off, v);
        }
      }
    }
    if (p.bcast) {
      __syncthreads();  // every thread's stores of this row precede the releases below
      if (threadIdx.x < p.ws && p.done[threadIdx.x] != nullptr) ptx::red_release_sys_add(p.done[threadIdx.x], 1u);
    } else if (p.norm) {
      __syncthreads();  // red_buf is reused by the next row
    }
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
