// Exact-mode linear for batches of more than 128 rows: the ACTIVATION rows on the MMA M side, on CTA pairs.
//
// exact_linear_kernel puts 128 weight rows on the MMA M side: a decode batch of 256 rows is then 6 activation tiles
// of 48 rows, every weight tile is staged into shared memory by 6 CTAs, and per 128-byte K block a CTA moves 66 KB
// through shared memory for 864 cycles of tensor work. It runs at about half of the tensor rate, bound by the bytes
// in flight towards shared memory, not by the math.
//
// Here a CTA pair (tcgen05 .cta_group::2, see limb_gemm_pair.cuh for the pair mechanics) covers 256 activation rows:
// each CTA holds 128 rows of the three activation limb planes as three A tiles, and the B operand of the pair is the
// three weight limbs of TN weight rows STACKED [W0 | W1 | W2] (N = 3 TN <= 240), half of it in each CTA. One MMA per
// activation limb i multiplies A_i [256 x 32] with all three weight limbs and accumulates into TMEM columns
// [i TN, (i + 3) TN): column block b = i + j again collects the limb products of weight 2^(8b). For a batch of up to
// 256 rows every weight byte is staged into exactly ONE CTA's shared memory (the weight stream is a single pass, as
// in a matrix-vector product), and a K block is 63 KB per CTA for 1440 cycles of tensor work at TN = 80.
//
// Epilogue: TMEM lane = activation row m (one thread per row), columns = weight rows. A thread joins the five
// blocks of 8 consecutive weight rows, adds the sparse residual of those rows (their lists are warp-uniform loads)
// and stores 8 consecutive int64 of its output row. Same integers as exact_linear_kernel.
#pragma once

#include "exact_linear.cuh"


namespace bx {

template <int TN, bool DBL>
struct RowsCfg {
  static_assert(TN % 16 == 0 && TN >= 16 && 3 * TN <= 256, "weight rows per tile: multiple of 16, 3 TN <= 256");
  static constexpr int COLS = 5 * TN;
  static constexpr int NBUF = DBL ? 2 : 1;
  static_assert(NBUF * COLS <= 512, "accumulators must fit in TMEM");
  static constexpr int USED = NBUF * COLS;
  static constexpr int TCOLS = USED <= 32 ? 32 : USED <= 64 ? 64 : USED <= 128 ? 128 : USED <= 256 ? 256 : 512;
  static constexpr int HALF = TN / 2;                       // weight rows per B chunk
  static constexpr int A_BYTES = 3 * WROWS * BKB;           // three activation limb tiles of 128 rows
  static constexpr int B_BYTES = 3 * HALF * BKB;            // this CTA's half of the stacked weight limbs
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_MAX = (227 * 1024 - 2048) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_MAX > 6 ? 6 : STAGES_MAX;
  static_assert(STAGES >= 2, "at least two stages");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512;
};

template <int TN>
struct RowsEpilogue {
  // Thread = activation row m0 + 32 quarter + lane; its group walks the tile's weight rows in chunks of CW = 4
  // (every tile size divides evenly among the EPI_GROUPS warps of a lane quarter; chunks of 8 spill registers).
  static constexpr int CW = 4;
  static constexpr int NS = (TN + 31) / 32;

  // Loaded before the accumulators are waited for: the thread's row exponent and, lane-held (lane_slot), the
  // constants of the tile's TN weight rows. No global load is left between the accumulator read-out and the stores,
  // except the gathers of the few weight rows with a residual list.
  struct Row {
    int m;
    bool mok;
    i64 shm;
    int d[NS], cnt[NS];
    i64 gd[NS];
  };

  static __device__ __forceinline__ Row load_row(int quarter, int lane, int n0, int m0, const ExactEpiParams& p) {
    Row r;
    r.m = m0 + quarter * 32 + lane;
    r.mok = r.m < p.M;
    r.shm = r.mok ? p.sh[r.m] : 0;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int c = s * 32 + lane, n = n0 + c;
      const bool nok = c < TN && n < p.N;
      r.d[s] = nok ? (int)__ldg(p.d + n) : 0;
      r.gd[s] = nok ? __ldg(p.g + n) - (i64)r.d[s] + FR : 0;
      r.cnt[s] = (nok && p.cnt) ? __ldg(p.cnt + n) : 0;
    }
    return r;
  }

  // One output chunk: constants by shuffle, residual, rounding, store. T: the joined accumulators of the chunk.
  static __device__ __forceinline__ void finish_chunk(const i64 (&T)[CW], int c0, int n0, const ExactEpiParams& p,
                                                      const Row& r, const int32_t* qrow, i64* yrow, bool vec,
                                                      bool& any_bad) {
    const int d_slot = lane_slot<NS>(r.d, c0), cnt_slot = lane_slot<NS>(r.cnt, c0);
    const i64 gd_slot = lane_slot<NS>(r.gd, c0);
    i64 out[CW];
#pragma unroll
    for (int i = 0; i < CW; ++i) {
      const int n = n0 + c0 + i, src = (c0 & 31) + i;
      const int dv = __shfl_sync(0xffffffffu, d_slot, src), cntv = __shfl_sync(0xffffffffu, cnt_slot, src);
      const i64 gdv = __shfl_sync(0xffffffffu, gd_slot, src);
      const bool on = n < p.N && r.mok;
      i64 B = 0;
      if (on)
        for (int j = 0; j < cntv; ++j)
          B += (i64)qrow[__ldg(p.ec + (i64)n * p.R + j)] * __ldg(p.ev + (i64)n * p.R + j);
      bool bad;
      out[i] = round_rule_warp(T[i], B, dv, r.shm + gdv, on, bad);
      any_bad |= bad;
    }
    if (r.mok) {
      if (vec && n0 + c0 + CW <= p.N) {                 // one full 32-byte sector per thread
        st_global_v4(yrow + n0 + c0, out[0], out[1], out[2], out[3]);
      } else {
#pragma unroll
        for (int i = 0; i < CW; ++i)
          if (n0 + c0 + i < p.N) yrow[n0 + c0 + i] = out[i];
      }
    }
  }

  static __device__ __forceinline__ void run(uint32_t tmem, int quarter, int group, int lane, int n0, int m0,
                                             const ExactEpiParams& p, const Row& r) {
    const int32_t* qrow = p.q + (i64)(r.mok ? r.m : 0) * p.ldq;
    i64* yrow = reinterpret_cast<i64*>(p.y) + (i64)(r.mok ? r.m : 0) * p.N;
    const bool vec = (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 31) == 0;
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
    bool any_bad = false;
#pragma unroll 1
    for (int c0 = group * CW; c0 < TN; c0 += CW * EPI_GROUPS) {
      if (n0 + c0 >= p.N) break;                     // warp-uniform
      uint32_t acc[5][CW];
#pragma unroll
      for (int b = 0; b < 5; ++b) tmem_ldn<CW>(tbase + b * TN + c0, acc[b]);
      tmem_ld_wait();
      i64 T[CW];
#pragma unroll
      for (int i = 0; i < CW; ++i) T[i] = join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]);
      finish_chunk(T, c0, n0, p, r, qrow, yrow, vec, any_bad);
    }
    if (p.checked && any_bad) *p.flag = 1;
  }

  // The two halves of run for a kernel with one accumulator buffer: drain reads the thread's accumulators out and
  // joins them (the buffer can be handed back right after), finish does the rest from registers.
  static constexpr int NCH = TN / (CW * EPI_GROUPS);
  struct Drained {
    i64 T[NCH][CW];
  };

  static __device__ __forceinline__ void drain(uint32_t tmem, int quarter, int group, int n0, const ExactEpiParams& p,
                                               Drained& a) {
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c0 = (k * EPI_GROUPS + group) * CW;
      if (n0 + c0 < p.N) {                           // warp-uniform
        uint32_t acc[5][CW];
#pragma unroll
        for (int b = 0; b < 5; ++b) tmem_ldn<CW>(tbase + b * TN + c0, acc[b]);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < CW; ++i) a.T[k][i] = join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]);
      }
    }
  }

  static __device__ __forceinline__ void finish(const Drained& a, int group, int n0, const ExactEpiParams& p,
                                                const Row& r) {
    const int32_t* qrow = p.q + (i64)(r.mok ? r.m : 0) * p.ldq;
    i64* yrow = reinterpret_cast<i64*>(p.y) + (i64)(r.mok ? r.m : 0) * p.N;
    const bool vec = (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 31) == 0;
    bool any_bad = false;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c0 = (k * EPI_GROUPS + group) * CW;
      if (n0 + c0 < p.N) finish_chunk(a.T[k], c0, n0, p, r, qrow, yrow, vec, any_bad);
    }
    if (p.checked && any_bad) *p.flag = 1;
  }
};

// The same layout on ONE CTA: the limb product is symmetric in its operands, so limb_gemm_persistent runs unchanged
// with the activation planes as its 128-row operand and TN weight rows as its stacked operand; only the epilogue
// (TMEM lane = activation row) differs. A batch of 256 rows is two row blocks without a ragged tile (six tiles of 48
// rows cover 288), and the residual lists, which belong to weight rows, are warp-uniform here. TN = 48: two
// accumulator buffers; TN = 64 / 80: one buffer (320 / 400 columns), wider MMAs, the epilogue not overlapped.
template <int TN>
struct RowsEpilogueOne {
  using Params = ExactEpiParams;
  using Row = typename RowsEpilogue<TN>::Row;
  // a0: first activation row of the tile (the 128-row operand), w0: first weight row (the stacked operand)
  static __device__ __forceinline__ Row load_row(int quarter, int, int lane, int a0, int w0, const Params& p) {
    return RowsEpilogue<TN>::load_row(quarter, lane, w0, a0, p);
  }
  static __device__ __forceinline__ void prefetch(const Row&, int, int, int, const Params&) {}
  static __device__ __forceinline__ void run(uint32_t tmem, int quarter, int group, int lane, int a0, int w0, bool,
                                             const Params& p, const Row& r) {
    RowsEpilogue<TN>::run(tmem, quarter, group, lane, w0, a0, p, r);
  }
  using Drained = typename RowsEpilogue<TN>::Drained;
  static __device__ __forceinline__ void drain(uint32_t tmem, int quarter, int group, int, int, int w0, bool,
                                               const Params& p, Drained& a) {
    RowsEpilogue<TN>::drain(tmem, quarter, group, w0, p, a);
  }
  static __device__ __forceinline__ void finish(const Drained& a, int, int group, int, int, int w0, const Params& p,
                                                const Row& r) {
    RowsEpilogue<TN>::finish(a, group, w0, p, r);
  }
};

template <int TN, int NBUF>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
exact_linear_rows_one_kernel(const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_wt,
                             const ExactEpiParams ep, int K, int row_blocks, int w_tiles) {
  limb_gemm_persistent<3, 3, TN, RowsEpilogueOne<TN>, NBUF, true>(&tmap_act, &tmap_wt, row_blocks, w_tiles,
                                                                  (K + BKB - 1) / BKB, ep);
}

// tmap_a: activation limb planes [3, M, K], boxes of 128 rows x 3 planes; tmap_w: weight limbs [3, N, K], boxes of
// TN / 2 rows of one plane. Tiles: n_tiles = ceil(N / TN) by m_tiles2 = ceil(M / 256), the batch index fastest.
template <int TN, bool DBL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
exact_linear_rows_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                         const ExactEpiParams ep, int K, int n_tiles, int m_tiles2) {
  using Cfg = RowsCfg<TN, DBL>;
  constexpr int EPI_WARPS = 4 * EPI_GROUPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PairShared* sh = reinterpret_cast<PairShared*>(ring + Cfg::STAGES * Cfg::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const uint32_t peer = rank ^ 1;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total = n_tiles * m_tiles2;
  const int nkb = (K + BKB - 1) / BKB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
      mbar_init(&sh->peer_full[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 2 * EPI_WARPS);
    }
    sh->abort_flag = *reinterpret_cast<volatile int*>(&g_wait_timeouts) != 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  __syncthreads();
  if (warp == 1) {                                   // each CTA allocates the same columns of its own SM's TMEM
    tmem_alloc(&sh->tmem_base, Cfg::TCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  cluster_arrive();
  cluster_wait();
  bool dead = sh->abort_flag != 0;
  {
    uint32_t other, other_abort;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other) : "r"(mapa_shared(smem_u32(&sh->tmem_base), peer)));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other_abort) : "r"(mapa_shared(smem_u32(&sh->abort_flag), peer)));
    if (other != tmem) {                             // one tensor-memory address must name both accumulators
      if (threadIdx.x == 0) atomicAdd(&g_wait_timeouts, 1);
      dead = true;
    }
    dead = dead || other_abort != 0;
  }
  cluster_arrive();
  cluster_wait();

  if (!dead) {
    if (warp == 0) {
      if (lane == 0) {
        // ---- TMA producer (both CTAs): own 128 activation rows (three limb tiles) + own half of the weight rows ----
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total && ok; tile += npairs) {
          const int n0 = (tile / m_tiles2) * TN, m0 = ((tile % m_tiles2) * 2 + (int)rank) * WROWS;
          for (int i = 0; i < nkb && ok; ++i, ++it) {
            const int s = it % Cfg::STAGES, round = it / Cfg::STAGES;
            if (round > 0) ok = mbar_wait(&sh->empty[s], (round - 1) & 1);
            if (!ok) break;
            uint8_t* st = ring + s * Cfg::STAGE_BYTES;
            mbar_arrive_expect_tx(&sh->full[s], Cfg::STAGE_BYTES);
#pragma unroll
            for (int c = 0; c < 3; ++c) {
              const int g = (int)rank * 3 + c;       // chunk g = 2 limb + half of the stacked weight rows
              tma_load_3d(st + Cfg::A_BYTES + c * Cfg::HALF * BKB, &tmap_w, &sh->full[s], i * BKB,
                          n0 + (g & 1) * Cfg::HALF, g >> 1);
            }
            tma_load_3d(st, &tmap_a, &sh->full[s], i * BKB, m0, 0);
          }
        }
        if (!ok) {
          atomicAdd(&g_wait_timeouts, 1);
          sh->abort_flag = 1;
          for (int i = (it > Cfg::STAGES ? it - Cfg::STAGES : 0); i < it; ++i)
            mbar_wait(&sh->full[i % Cfg::STAGES], (i / Cfg::STAGES) & 1);
        }
      }
    } else if (warp == 1) {
      if (lane == 0 && rank != 0) {
        // ---- peer: tell the leader when a stage of this CTA has landed ----
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total && ok; tile += npairs)
          for (int i = 0; i < nkb && ok; ++i, ++it) {
            const int s = it % Cfg::STAGES;
            ok = mbar_wait(&sh->full[s], (it / Cfg::STAGES) & 1);
            if (ok) mbar_arrive_cluster(mapa_shared(smem_u32(&sh->peer_full[s]), 0));
          }
        if (!ok) {
          atomicAdd(&g_wait_timeouts, 1);
          sh->abort_flag = 1;
        }
      } else if (lane == 0) {
        // ---- leader: MMA issue for the pair ----
        constexpr uint32_t ID_ALL = umma_idesc_i8_pair(3 * TN);
        int it = 0, tcount = 0;
        bool ok = true;
        for (int tile = pair; tile < total && ok; tile += npairs, ++tcount) {
          const int buf = DBL ? (tcount & 1) : 0, use = DBL ? (tcount >> 1) : tcount;
          ok = mbar_wait_cluster(&sh->acc_empty[buf], use & 1);      // drained and cleared by both CTAs' epilogues
          if (!ok) break;
          tc_fence_after();
          const uint32_t acc = tmem + buf * Cfg::COLS;
          for (int i = 0; i < nkb && ok; ++i, ++it) {
            const int s = it % Cfg::STAGES;
            const uint32_t par = (it / Cfg::STAGES) & 1;
            ok = mbar_wait(&sh->full[s], par) && mbar_wait_cluster(&sh->peer_full[s], par);
            if (!ok) break;
            tc_fence_after();
            const uint32_t abase = smem_u32(ring + s * Cfg::STAGE_BYTES);
            const uint32_t bbase = abase + Cfg::A_BYTES;
#pragma unroll
            for (int ks = 0; ks < BKB / UMMA_K; ++ks) {
              const uint32_t koff = ks * UMMA_K;
              const uint64_t bdesc = umma_desc_sw128(bbase + koff);
#pragma unroll
              for (int l = 0; l < 3; ++l)
                umma_i8_pair(acc + l * TN, umma_desc_sw128(abase + l * (WROWS * BKB) + koff), bdesc, ID_ALL,
                             (i == 0 && ks == 0 && l == 0) ? 0u : 1u);
            }
            umma_commit_pair(smem_u32(&sh->empty[s]));
            umma_commit_pair(mapa_shared(smem_u32(&sh->empty[s]), 1));
          }
          if (ok) {
            umma_commit_pair(smem_u32(&sh->acc_full[buf]));
            umma_commit_pair(mapa_shared(smem_u32(&sh->acc_full[buf]), 1));
          }
        }
        if (!ok) {
          atomicAdd(&g_wait_timeouts, 1);
          sh->abort_flag = 1;
        }
      }
    } else {
      // ---- epilogue warps (both CTAs): own 128 activation rows ----
      const int quarter = warp & 3, group = (warp - 2) >> 2;
      const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
      const uint32_t acc_empty0 = mapa_shared(smem_u32(&sh->acc_empty[0]), 0);
      const uint32_t acc_empty1 = mapa_shared(smem_u32(&sh->acc_empty[1]), 0);
      auto hand_back = [&](int buf) {
        // Blocks 3 and 4 are only ever accumulated into: they start every tile at zero. A warp clears exactly the
        // columns it reads in RowsEpilogue::run, so no warp clears what another still reads.
        constexpr int CW = RowsEpilogue<TN>::CW;
        for (int c0 = group * CW; c0 < TN; c0 += CW * EPI_GROUPS) {
#pragma unroll
          for (int b = 3; b < 5; ++b) {
            const uint32_t at = tmem + lane_base + buf * Cfg::COLS + b * TN + c0;
            if constexpr (CW == 8) tmem_st8_fill(at, 0u); else tmem_st4_fill(at, 0u);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(buf ? acc_empty1 : acc_empty0);
      };
      hand_back(0);
      if (DBL) hand_back(1);
      int tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < total; tile += npairs, ++tcount) {
        const int buf = DBL ? (tcount & 1) : 0, use = DBL ? (tcount >> 1) : tcount;
        const int w0 = (tile / m_tiles2) * TN, a0 = ((tile % m_tiles2) * 2 + (int)rank) * WROWS;
        const typename RowsEpilogue<TN>::Row row = RowsEpilogue<TN>::load_row(quarter, lane, w0, a0, ep);
        if (ok) ok = mbar_wait(&sh->acc_full[buf], use & 1);
        ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag) == 0);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        RowsEpilogue<TN>::run(tmem + buf * Cfg::COLS, quarter, group, lane, w0, a0, ep, row);
        hand_back(buf);
      }
      if (!ok && lane == 0) atomicAdd(&g_wait_timeouts, 1);
    }
  }

  // Every thread of both CTAs: no remote arrival, commit or operand read may target a CTA that has left.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TCOLS);
  }
}

}  // namespace bx
