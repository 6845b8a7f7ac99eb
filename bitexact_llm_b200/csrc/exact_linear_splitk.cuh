// Split-K form of the exact-mode linear for small batches (M <= 128) on projections with few weight tiles.
//
// With one CTA per 128 weight rows, the down projection (N = 2048, K = 8192) has 16 CTAs: 16 of 148 SMs stream the
// 50 MB of weight limbs and a batch-1 decode step runs at a fraction of the HBM rate. Here a thread-block CLUSTER of S
// CTAs shares an output tile: CTA `rank` runs the tcgen05 main loop of limb_gemm.cuh over its slice of the K blocks;
// the int32 limb sums of the slices are joined to int64 in each CTA and reduce-scattered through distributed shared
// memory: activation row (accumulator column) c of the tile belongs to CTA c mod S, every CTA stores its partial sums
// of column c into that CTA's idle TMA ring (st.shared::cluster, between two cluster barriers), and every CTA adds
// the S partial columns it owns (integer sums: exact in any order) and runs the usual epilogue on them (sparse
// residual, one rounding, flag). The tail of the kernel is shared by the S CTAs instead of falling on one.
// Same integers as exact_linear_kernel.
#pragma once

#include <cooperative_groups.h>

#include "exact_linear.cuh"

namespace bx {

constexpr int SPLITK_MAX = 8;

// Most K slices a tile of TA activation rows can take: a CTA's ring holds S partial copies of its ceil(TA / S)
// columns (128 int64 each), at most (TA + S - 1) x 1 KB.
template <int TA>
__host__ __device__ constexpr int splitk_limit() {
  using Cfg = GemmCfg<3, 3, TA>;
  static_assert((TA + SPLITK_MAX - 1) * WROWS * 8 <= Cfg::STAGES * Cfg::STAGE_BYTES, "partial columns fit in the ring");
  return SPLITK_MAX;
}

template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
exact_linear_splitk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                           const ExactEpiParams ep, int K, int m_tiles) {
  namespace cg = cooperative_groups;
  using Cfg = GemmCfg<3, 3, TA>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmShared* sh = reinterpret_cast<GemmShared*>(ring + Cfg::STAGES * Cfg::STAGE_BYTES);
  i64* partial = reinterpret_cast<i64*>(ring);                        // after the main loops: [S sources][owned column][128]

  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int tile = blockIdx.x / S;
  const int m0 = (tile % m_tiles) * TA;
  const int n0 = (tile / m_tiles) * WROWS;
  const int nkb_all = (K + BKB - 1) / BKB;
  const int kb0 = (int)(((int64_t)rank * nkb_all) / S), kb1 = (int)(((int64_t)(rank + 1) * nkb_all) / S);
  const int nkb = kb1 - kb0;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    mbar_init(&sh->acc_full, 1);
    // A timeout anywhere earlier (sticky until the host clears it): no CTA starts its main loop, but every CTA still
    // walks through the cluster barriers below, so none is left waiting.
    sh->abort_flag = *reinterpret_cast<volatile int*>(&g_wait_timeouts) != 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_a);
  }
  __syncthreads();
  const bool dead = sh->abort_flag != 0;
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  bool acc_ok = false;                                                // epilogue warps: accumulators complete
  // epilogue threads: constants of weight row n (see ExactEpilogue), loaded before the accumulators exist
  constexpr int RMAX = 2;
  bool nok = false;
  int d = 0, cnt = 0, wcnt = 0;
  i64 gd = 0;
  int ecr[RMAX] = {0, 0};
  i64 evr[RMAX] = {0, 0};
  constexpr int NS = (TA + 31) / 32;
  i64 shv[NS];                                                        // the tile's row exponents, lane-held
#pragma unroll
  for (int s = 0; s < NS; ++s) shv[s] = 0;

  if (warp == 0) {
    if (lane == 0 && !dead) {
      // ---- TMA producer ----
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % Cfg::STAGES;
        const int round = i / Cfg::STAGES;
        if (round > 0) ok = mbar_wait(&sh->empty[s], (round - 1) & 1);
        if (!ok) break;
        uint8_t* st = ring + s * Cfg::STAGE_BYTES;
        mbar_arrive_expect_tx(&sh->full[s], Cfg::STAGE_BYTES);
        tma_load_3d(st, &tmap_w, &sh->full[s], (kb0 + i) * BKB, n0, 0);
        tma_load_3d(st + Cfg::W_BYTES, &tmap_a, &sh->full[s], (kb0 + i) * BKB, m0, 0);
        issued = i + 1;
      }
      if (!ok) {
        atomicAdd(&g_wait_timeouts, 1);
        sh->abort_flag = 1;
        for (int i = (issued > Cfg::STAGES ? issued - Cfg::STAGES : 0); i < issued; ++i)
          mbar_wait(&sh->full[i % Cfg::STAGES], (i / Cfg::STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && !dead) {
      // ---- MMA issue (as limb_gemm_tile) ----
      constexpr uint32_t ID_ALL = umma_idesc_i8(3 * TA);
      constexpr uint32_t ID_ONE = umma_idesc_i8(TA);
      constexpr uint32_t ID_REST = umma_idesc_i8(2 * TA);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % Cfg::STAGES;
        ok = mbar_wait(&sh->full[s], (i / Cfg::STAGES) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t wbase = smem_u32(ring + s * Cfg::STAGE_BYTES);
        const uint32_t abase = wbase + Cfg::W_BYTES;
#pragma unroll
        for (int ks = 0; ks < BKB / UMMA_K; ++ks) {
          const uint32_t koff = ks * UMMA_K;
          const uint64_t adesc = umma_desc_sw128(abase + koff);
          if (i == 0 && ks == 0) {
            umma_i8(tmem, umma_desc_sw128(wbase + koff), adesc, ID_ALL, 0);
#pragma unroll
            for (int j = 1; j < 3; ++j) {
              const uint64_t wdesc = umma_desc_sw128(wbase + j * (WROWS * BKB) + koff);
              umma_i8(tmem + (j + 2) * TA, wdesc, umma_desc_sw128(abase + 2 * TA * BKB + koff), ID_ONE, 0);
              umma_i8(tmem + j * TA, wdesc, adesc, ID_REST, 1);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 3; ++j)
              umma_i8(tmem + j * TA, umma_desc_sw128(wbase + j * (WROWS * BKB) + koff), adesc, ID_ALL, 1);
          }
        }
        umma_commit(&sh->empty[s]);
      }
      if (ok) {
        umma_commit(&sh->acc_full);
      } else {
        atomicAdd(&g_wait_timeouts, 1);
        sh->abort_flag = 1;
      }
    }
  } else {
    // ---- epilogue warps: the per-row constants and the residual list of weight row n do not depend on the
    //      accumulators; at decode sizes this kernel is a latency chain, so their loads start before the wait ----
    {
      const int n = n0 + (warp & 3) * 32 + lane;
      nok = n < ep.N;
      d = nok ? (int)ep.d[n] : 0;
      gd = nok ? ep.g[n] - (i64)d + FR : 0;
      cnt = (nok && ep.cnt) ? ep.cnt[n] : 0;
#pragma unroll
      for (int j = 0; j < RMAX; ++j) {
        if (j < cnt) {
          ecr[j] = ep.ec[(i64)n * ep.R + j];
          evr[j] = ep.ev[(i64)n * ep.R + j];
        }
      }
      wcnt = __reduce_max_sync(0xffffffffu, cnt);                      // longest list in the warp (uniform)
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int c = s * 32 + lane;
        if (c < TA && m0 + c < ep.M) shv[s] = ep.sh[m0 + c];
      }
    }
    // ---- epilogue warps: wait for this CTA's accumulators ----
    bool ok = !dead;
    if (ok && nkb > 0) ok = mbar_wait(&sh->acc_full, 0);
    ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag) == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) tc_fence_after();
    else if (lane == 0 && !dead) atomicAdd(&g_wait_timeouts, 1);
    acc_ok = ok && nkb > 0;
  }

  // Every CTA of the cluster has finished its main loop: the rings are idle and can take the partial columns.
  tc_fence_before();
  __syncthreads();
  cluster.sync();

  const int quarter = warp & 3, group = (warp - 2) >> 2;
  const int row = quarter * 32 + lane;                                // TMEM lane = weight row of the tile
  const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
  const int own = (TA + S - 1) / S;                                   // columns a CTA owns at most
  if (warp >= 2) {
    // ---- join this CTA's limb sums and send column c to CTA c mod S, slot [this rank][c / S] ----
#pragma unroll 1
    for (int c0 = group * 8; c0 < TA; c0 += 8 * EPI_GROUPS) {
      if (m0 + c0 >= ep.M) break;
      uint32_t acc[5][8];
      if (acc_ok) {
#pragma unroll
        for (int b = 0; b < 5; ++b) tmem_ld8(tbase + b * TA + c0, acc[b]);
        tmem_ld_wait();
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i;
        if (m0 + c >= ep.M) break;
        const i64 T = acc_ok ? join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]) : 0;
        i64* dst = cluster.map_shared_rank(partial, c % S);
        dst[((size_t)rank * own + c / S) * WROWS + row] = T;
      }
    }
  }
  cluster.sync();                                                     // every partial column is in its owner's ring

  if (warp >= 2) {
    // ---- the columns this CTA owns: sum of the S partials, then the epilogue of exact_linear_kernel ----
    const int n = n0 + row;
    bool any_bad = false;
    for (int k = group; k < own; k += EPI_GROUPS) {
      const int c = rank + k * S;
      const int m = m0 + c;
      if (c >= TA || m >= ep.M) break;                                // warp-uniform
      i64 T = 0;
      for (int r = 0; r < S; ++r) T += partial[((size_t)r * own + k) * WROWS + row];
      i64 B = 0;
      if (wcnt > 0 && nok) {
#pragma unroll
        for (int j = 0; j < RMAX; ++j)
          if (j < wcnt && j < cnt) B += (i64)ep.q[(i64)m * ep.ldq + ecr[j]] * evr[j];
        for (int j = RMAX; j < cnt; ++j)
          B += (i64)ep.q[(i64)m * ep.ldq + ep.ec[(i64)n * ep.R + j]] * ep.ev[(i64)n * ep.R + j];
      }
      const i64 pv = __shfl_sync(0xffffffffu, lane_slot<NS>(shv, c), c & 31) + gd;
      bool bad;
      const i64 yv = round_rule_warp(T, B, d, pv, nok, bad);
      any_bad |= bad;
      if (nok) ep.y[(i64)m * ep.N + n] = yv;
    }
    if (ep.checked && any_bad) *ep.flag = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

}  // namespace bx
