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

// The exact-mode policy of limb_splitk: what an epilogue thread knows about its weight row before the accumulators
// exist, how the column blocks join, and the tail (sparse residual, one rounding, flag) of an owned output.
template <int TA>
struct ExactSplitEpi {
  using Params = ExactEpiParams;
  static constexpr int NW = 3, NA = 3, RMAX = 2, NS = (TA + 31) / 32;
  struct Consts {
    int n, d, cnt, wcnt;
    bool nok;
    i64 gd;
    int ecr[RMAX];
    i64 evr[RMAX];
    i64 shv[NS];                                                      // the tile's row exponents, lane-held
  };

  static __device__ __forceinline__ Consts load(int n0, int m0, int quarter, int group, int lane, int rank, int S,
                                                const Params& ep) {
    Consts c;
    c.n = n0 + quarter * 32 + lane;
    c.nok = c.n < ep.N;
    c.d = c.nok ? (int)ep.d[c.n] : 0;
    c.gd = c.nok ? ep.g[c.n] - (i64)c.d + FR : 0;
    c.cnt = (c.nok && ep.cnt) ? ep.cnt[c.n] : 0;
#pragma unroll
    for (int j = 0; j < RMAX; ++j) {
      c.ecr[j] = 0;
      c.evr[j] = 0;
      if (j < c.cnt) {
        c.ecr[j] = ep.ec[(i64)c.n * ep.R + j];
        c.evr[j] = ep.ev[(i64)c.n * ep.R + j];
      }
    }
    c.wcnt = __reduce_max_sync(0xffffffffu, c.cnt);                    // longest list in the warp (uniform)
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int col = s * 32 + lane;
      c.shv[s] = (col < TA && m0 + col < ep.M) ? ep.sh[m0 + col] : 0;
    }
    return c;
  }

  static __device__ __forceinline__ i64 join(const uint32_t (&acc)[5][8], int i) {
    return join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]);
  }
  static __device__ __forceinline__ int a_rows(const Params& ep) { return ep.M; }   // rows of the stacked operand

  // Output (m, c.n) of tile column col from the summed limb sums T. All 32 lanes of a warp call it together.
  // (Dealing the outputs of rows with a residual list out over the warp, as exact_linear_kernel does, was measured
  // here too: nothing at 256 rows, 0.7 us slower at 1 .. 16 rows.)
  static __device__ __forceinline__ void final(i64 T, int col, int m, const Consts& c, const Params& ep, bool& any_bad) {
    i64 B = 0;
    if (c.wcnt > 0 && c.nok) {
#pragma unroll
      for (int j = 0; j < RMAX; ++j)
        if (j < c.wcnt && j < c.cnt) B += (i64)ep.q[(i64)m * ep.ldq + c.ecr[j]] * c.evr[j];
      for (int j = RMAX; j < c.cnt; ++j)
        B += (i64)ep.q[(i64)m * ep.ldq + ep.ec[(i64)c.n * ep.R + j]] * ep.ev[(i64)c.n * ep.R + j];
    }
    const i64 pv = __shfl_sync(0xffffffffu, lane_slot<NS>(c.shv, col), col & 31) + c.gd;
    bool bad;
    const i64 yv = round_rule_warp(T, B, c.d, pv, c.nok, bad);
    any_bad |= bad;
    if (c.nok) ep.y[(i64)m * ep.N + c.n] = yv;
  }

  static __device__ __forceinline__ void finish(bool any_bad, const Params& ep) {
    if (ep.checked && any_bad) *ep.flag = 1;
  }
};

template <int TA, class Epi>
__device__ __forceinline__ void limb_splitk(const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                                            const typename Epi::Params& ep, int K, int m_tiles) {
  namespace cg = cooperative_groups;
  constexpr int NW = Epi::NW, NA = Epi::NA, NBLK = NW + NA - 1;
  using Cfg = GemmCfg<NW, NA, TA>;
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
  typename Epi::Consts cst = {};                                     // epilogue threads: loaded before the wait

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
      constexpr uint32_t ID_ALL = umma_idesc_i8(NA * TA);
      constexpr uint32_t ID_ONE = umma_idesc_i8(TA);
      constexpr uint32_t ID_REST = umma_idesc_i8(NA > 1 ? (NA - 1) * TA : TA);
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
            for (int j = 1; j < NW; ++j) {
              const uint64_t wdesc = umma_desc_sw128(wbase + j * (WROWS * BKB) + koff);
              umma_i8(tmem + (j + NA - 1) * TA, wdesc, umma_desc_sw128(abase + (NA - 1) * TA * BKB + koff), ID_ONE, 0);
              if (NA > 1) umma_i8(tmem + j * TA, wdesc, adesc, ID_REST, 1);
            }
          } else {
#pragma unroll
            for (int j = 0; j < NW; ++j)
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
    // ---- epilogue warps: what does not depend on the accumulators (per-row constants, lists, row scales) is loaded
    //      first; at decode sizes this kernel is a latency chain ----
    cst = Epi::load(n0, m0, warp & 3, (warp - 2) >> 2, lane, rank, S, ep);
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
      if (m0 + c0 >= Epi::a_rows(ep)) break;
      uint32_t acc[NBLK][8];
      if (acc_ok) {
#pragma unroll
        for (int b = 0; b < NBLK; ++b) tmem_ld8(tbase + b * TA + c0, acc[b]);
        tmem_ld_wait();
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i;
        if (m0 + c >= Epi::a_rows(ep)) break;
        const i64 T = acc_ok ? Epi::join(acc, i) : 0;
        i64* dst = cluster.map_shared_rank(partial, c % S);
        dst[((size_t)rank * own + c / S) * WROWS + row] = T;
      }
    }
  }
  cluster.sync();                                                     // every partial column is in its owner's ring

  if (warp >= 2) {
    // ---- the columns this CTA owns: sum of the S partials, then the usual tail of the epilogue ----
    bool any_bad = false;
    for (int k = group; k < own; k += EPI_GROUPS) {
      const int c = rank + k * S;
      const int m = m0 + c;
      if (c >= TA || m >= Epi::a_rows(ep)) break;                     // warp-uniform
      i64 T = 0;
      for (int r = 0; r < S; ++r) T += partial[((size_t)r * own + k) * WROWS + row];
      Epi::final(T, c, m, cst, ep, any_bad);
    }
    Epi::finish(any_bad, ep);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// The exact-mode policy with the ACTIVATION rows as the 128-row operand (TMEM lane = activation row) and TA weight
// rows as the stacked operand: the residual lists then belong to accumulator columns, a warp takes the list branch
// together, and only the few listed columns pay for a gather (down projection at 256 rows, weight-major: 40.7 us
// with the lists against 32.8 us without). In limb_splitk's terms n0 is the first activation row of the tile and
// the stacked-operand rows (m0 + column) are weight rows.
template <int TA>
struct ExactRowsSplitEpi {
  using Params = ExactEpiParams;
  static constexpr int NW = 3, NA = 3, NS = (TA + 31) / 32;
  struct Consts {
    int m;                                                            // this lane's activation row
    bool mok;
    i64 shm;
    int d[NS], cnt[NS], ec0[NS];                                      // the tile's weight rows, lane-held
    i64 gd[NS], ev0[NS];                                              // (ec0, ev0: first entry of the row's list)
  };

  static __device__ __forceinline__ Consts load(int a0, int w0, int quarter, int, int lane, int, int, const Params& ep) {
    Consts c;
    c.m = a0 + quarter * 32 + lane;
    c.mok = c.m < ep.M;
    c.shm = c.mok ? ep.sh[c.m] : 0;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int col = s * 32 + lane, n = w0 + col;
      const bool nok = col < TA && n < ep.N;
      c.d[s] = nok ? (int)__ldg(ep.d + n) : 0;
      c.gd[s] = nok ? __ldg(ep.g + n) - (i64)c.d[s] + FR : 0;
      c.cnt[s] = (nok && ep.cnt) ? __ldg(ep.cnt + n) : 0;
      c.ec0[s] = c.cnt[s] > 0 ? __ldg(ep.ec + (i64)n * ep.R) : 0;
      c.ev0[s] = c.cnt[s] > 0 ? __ldg(ep.ev + (i64)n * ep.R) : 0;
    }
    return c;
  }

  static __device__ __forceinline__ i64 join(const uint32_t (&acc)[5][8], int i) {
    return join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]);
  }
  static __device__ __forceinline__ int a_rows(const Params& ep) { return ep.N; }

  // Output (c.m, n) from the summed limb sums T; n = weight row (warp-uniform), col = its column in the tile.
  static __device__ __forceinline__ void final(i64 T, int col, int n, const Consts& c, const Params& ep, bool& any_bad) {
    const int src = col & 31;
    const int d = __shfl_sync(0xffffffffu, lane_slot<NS>(c.d, col), src);
    const int cnt = __shfl_sync(0xffffffffu, lane_slot<NS>(c.cnt, col), src);
    const i64 gd = __shfl_sync(0xffffffffu, lane_slot<NS>(c.gd, col), src);
    i64 B = 0;
    if (cnt > 0) {                                                    // warp-uniform
      const int ec0 = __shfl_sync(0xffffffffu, lane_slot<NS>(c.ec0, col), src);
      const i64 ev0 = __shfl_sync(0xffffffffu, lane_slot<NS>(c.ev0, col), src);
      if (c.mok) {
        B = (i64)ep.q[(i64)c.m * ep.ldq + ec0] * ev0;
        for (int j = 1; j < cnt; ++j)
          B += (i64)ep.q[(i64)c.m * ep.ldq + __ldg(ep.ec + (i64)n * ep.R + j)] * __ldg(ep.ev + (i64)n * ep.R + j);
      }
    }
    bool bad;
    const i64 yv = round_rule_warp(T, B, d, c.shm + gd, c.mok, bad);
    any_bad |= bad;
    if (c.mok) ep.y[(i64)c.m * ep.N + n] = yv;
  }

  static __device__ __forceinline__ void finish(bool any_bad, const Params& ep) {
    if (ep.checked && any_bad) *ep.flag = 1;
  }
};

template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
exact_linear_splitk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                           const ExactEpiParams ep, int K, int m_tiles) {
  limb_splitk<TA, ExactSplitEpi<TA>>(tmap_w, tmap_a, ep, K, m_tiles);
}

// tmap_act: activation limb planes (boxes of 128 rows), tmap_wt: weight limbs (boxes of TA rows); w_tiles = ceil(N / TA).
template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
exact_linear_rows_splitk_kernel(const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_wt,
                                const ExactEpiParams ep, int K, int w_tiles) {
  limb_splitk<TA, ExactRowsSplitEpi<TA>>(tmap_act, tmap_wt, ep, K, w_tiles);
}

}  // namespace bx
