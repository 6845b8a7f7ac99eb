// Limb GEMM main loop on CTA PAIRS (tcgen05 .cta_group::2): two CTAs on the two SMs of a TPC share one MMA.
//
// Why: with one CTA per tile the kernel is bound by shared-memory traffic, not by the tensor pipe. Per K slice an MMA
// reads its A operand (128 weight rows x 32 bytes) and its B operand (the NA stacked activation limb tiles) from
// shared memory while TMA writes the next stage into it; at TA = 48 that is 120 + 76 bytes per clock against a port
// of 128. In a pair, each CTA supplies 128 weight rows (the pair covers 256) and only HALF of the B operand: the
// hardware reads the first N / 2 rows of B from the leader's shared memory and the other half from the peer's. Per SM
// the B reads and the activation TMA traffic halve, the weight traffic per MAC is unchanged.
//
// Layout. Pair p = cluster of CTAs (2p, 2p + 1); cluster rank 0 is the leader and issues every MMA. A tile is 256
// weight rows x TA activation rows: CTA `rank` owns weight rows n0 + 128 rank .. + 127 (its TMA loads them into its
// own ring, its TMEM holds their accumulators, its epilogue warps store them). The B operand of an MMA is the
// NA * TA stacked limb rows [limb 0 | limb 1 | ...]; row r < NA TA / 2 lives in the leader, the rest in the peer.
// With chunks of TA / 2 rows, chunk g = 2 limb + half goes to CTA g / NA at chunk slot g % NA; one TMA box
// (128 bytes x TA / 2 rows) per chunk. Column block b = i + j of the accumulators, the first-slice rule and the
// epilogue are those of limb_gemm.cuh; the column blocks an accumulate-free first MMA cannot reach are cleared by
// the epilogue warps when they hand a buffer back.
//
// Hand-overs. Each CTA has its own TMA producer and full / empty barriers. The peer's warp 1 relays "stage landed"
// to the leader (remote mbarrier arrival); the leader waits for both, issues the MMAs and commits twice per stage:
// to its own `empty` barrier and to the peer's. Accumulator buffers (two, so the epilogue of tile i overlaps the MMAs
// of tile i + 1): `acc_full` is committed to both CTAs, `acc_empty` lives in the leader and counts the epilogue warps
// of both CTAs. No multicast of any kind. Every wait is bounded; all threads of both CTAs reach the closing cluster
// barrier on every path, so neither CTA can leave while the other may still touch its shared memory.
#pragma once

#include "limb_gemm.cuh"

namespace bx {

template <int NW, int NA, int TA>
struct PairCfg {
  static_assert(TA % 16 == 0 && TA >= 16, "activation tile: multiple of 16 rows (half tiles of whole swizzle atoms)");
  static_assert(NA * TA <= 256, "MMA N limit");
  static constexpr int NBLK = NW + NA - 1;
  static constexpr int COLS = NBLK * TA;
  static_assert(2 * COLS <= 512, "two accumulator buffers must fit in TMEM");
  static constexpr int TCOLS = 2 * COLS <= 64 ? 64 : 2 * COLS <= 128 ? 128 : 2 * COLS <= 256 ? 256 : 512;
  static constexpr int HALF = TA / 2;                       // rows per B chunk
  static constexpr int W_BYTES = NW * WROWS * BKB;
  static constexpr int B_BYTES = NA * HALF * BKB;           // this CTA's half of the B operand
  static constexpr int STAGE_BYTES = W_BYTES + B_BYTES;
  static constexpr int STAGES_MAX = (227 * 1024 - 2048) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_MAX > 6 ? 6 : STAGES_MAX;
  static_assert(STAGES >= 2, "at least two stages");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512;
  static constexpr int ZERO_COL0 = NA * TA;                 // columns [ZERO_COL0, COLS) start every tile at zero
};

struct PairShared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t peer_full[8];      // leader: the peer's stage has landed (relayed)
  uint64_t acc_full[2];
  uint64_t acc_empty[2];      // leader: count = epilogue warps of both CTAs
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int NW, int NA, int TA, class Epi>
__device__ __forceinline__ void limb_gemm_pair_persistent(const CUtensorMap* tmap_w, const CUtensorMap* tmap_b,
                                                          int n_tiles2, int m_tiles, int nkb,
                                                          const typename Epi::Params& ep) {
  using Cfg = PairCfg<NW, NA, TA>;
  constexpr int EPI_WARPS = 4 * EPI_GROUPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PairShared* sh = reinterpret_cast<PairShared*>(ring + Cfg::STAGES * Cfg::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const uint32_t peer = rank ^ 1;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total = n_tiles2 * m_tiles;

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
    tma_prefetch_desc(tmap_w);
    tma_prefetch_desc(tmap_b);
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
  // Both CTAs' barriers are initialised and both TMEM allocations exist before anything crosses the pair.
  cluster_arrive();
  cluster_wait();
  // The pair MMA addresses both accumulators with ONE tensor-memory address: the two allocations must coincide.
  bool dead = sh->abort_flag != 0;
  {
    uint32_t other;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other) : "r"(mapa_shared(smem_u32(&sh->tmem_base), peer)));
    uint32_t other_abort;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other_abort) : "r"(mapa_shared(smem_u32(&sh->abort_flag), peer)));
    if (other != tmem) {
      if (threadIdx.x == 0) atomicAdd(&g_wait_timeouts, 1);
      dead = true;
    }
    dead = dead || other_abort != 0;
  }
  // Nobody writes abort_flag between the cluster barrier above and the one below, so both CTAs read the same values.
  cluster_arrive();
  cluster_wait();

  if (!dead) {
    if (warp == 0) {
      if (lane == 0) {
        // ---- TMA producer (both CTAs): own 128 weight rows + own half of the B operand ----
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total && ok; tile += npairs) {
          const int n0 = ((tile / m_tiles) * 2 + (int)rank) * WROWS, m0 = (tile % m_tiles) * TA;
          for (int i = 0; i < nkb && ok; ++i, ++it) {
            const int s = it % Cfg::STAGES, round = it / Cfg::STAGES;
            if (round > 0) ok = mbar_wait(&sh->empty[s], (round - 1) & 1);
            if (!ok) break;
            uint8_t* st = ring + s * Cfg::STAGE_BYTES;
            mbar_arrive_expect_tx(&sh->full[s], Cfg::STAGE_BYTES);
            tma_load_3d(st, tmap_w, &sh->full[s], i * BKB, n0, 0);
#pragma unroll
            for (int c = 0; c < NA; ++c) {
              const int g = (int)rank * NA + c;      // chunk g = 2 limb + half
              tma_load_3d(st + Cfg::W_BYTES + c * Cfg::HALF * BKB, tmap_b, &sh->full[s], i * BKB,
                          m0 + (g & 1) * Cfg::HALF, g >> 1);
            }
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
        constexpr uint32_t ID_ALL = umma_idesc_i8_pair(NA * TA);
        int it = 0, tcount = 0;
        bool ok = true;
        for (int tile = pair; tile < total && ok; tile += npairs, ++tcount) {
          const int buf = tcount & 1, use = tcount >> 1;
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
            const uint32_t wbase = smem_u32(ring + s * Cfg::STAGE_BYTES);
            const uint32_t bbase = wbase + Cfg::W_BYTES;
#pragma unroll
            for (int ks = 0; ks < BKB / UMMA_K; ++ks) {
              const uint32_t koff = ks * UMMA_K;
              const uint64_t bdesc = umma_desc_sw128(bbase + koff);
#pragma unroll
              for (int j = 0; j < NW; ++j)
                umma_i8_pair(acc + j * TA, umma_desc_sw128(wbase + j * (WROWS * BKB) + koff), bdesc, ID_ALL,
                             (i == 0 && ks == 0 && j == 0) ? 0u : 1u);
            }
            umma_commit_pair(smem_u32(&sh->empty[s]));                       // both rings: stage free once read
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
      // ---- epilogue warps (both CTAs): own 128 accumulator lanes ----
      const int quarter = warp & 3, group = (warp - 2) >> 2;
      const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
      const uint32_t acc_empty0 = mapa_shared(smem_u32(&sh->acc_empty[0]), 0);
      const uint32_t acc_empty1 = mapa_shared(smem_u32(&sh->acc_empty[1]), 0);
      auto hand_back = [&](int buf) {
        // Column blocks no accumulate-free MMA writes start the next tile at zero. A warp clears exactly the columns
        // it reads in Epi::run (the chunks of Epi::CW activation rows of its group), so no warp clears what another still reads.
        if (Cfg::ZERO_COL0 < Cfg::COLS) {
          for (int c0 = group * Epi::CW; c0 < TA; c0 += Epi::CW * EPI_GROUPS)
#pragma unroll
            for (int b = NA; b < Cfg::NBLK; ++b) {
              const uint32_t at = tmem + lane_base + buf * Cfg::COLS + b * TA + c0;
              if constexpr (Epi::CW == 8) tmem_st8_fill(at, 0u); else tmem_st4_fill(at, 0u);
            }
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(buf ? acc_empty1 : acc_empty0);
      };
      hand_back(0);
      hand_back(1);
      int tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < total; tile += npairs, ++tcount) {
        const int buf = tcount & 1, use = tcount >> 1;
        const int n0 = ((tile / m_tiles) * 2 + (int)rank) * WROWS, m0 = (tile % m_tiles) * TA;
        const typename Epi::Row row = Epi::load_row(quarter, group, lane, n0, m0, ep);      // overlaps the tile's MMAs
        Epi::prefetch(row, group, lane, m0, ep);
        if (ok) ok = mbar_wait(&sh->acc_full[buf], use & 1);
        ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag) == 0);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        Epi::run(tmem + buf * Cfg::COLS, quarter, group, lane, n0, m0, nkb > 0, ep, row);
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
