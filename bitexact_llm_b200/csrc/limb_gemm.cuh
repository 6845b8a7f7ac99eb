// Limb GEMM main loop on tcgen05 (kind::i8) with TMEM accumulators, shared by the exact-mode linear
// (3 weight limbs x 3 activation limbs) and the int8-mode linear (1 weight limb x 2 activation limbs).
//
// Orientation: the WEIGHT rows are the MMA M side (128 rows per CTA = 128 TMEM lanes), the activation rows are
// the MMA N side (TA rows per limb). The NA activation limb tiles of one K block sit back to back in shared
// memory, so one MMA per weight limb j multiplies W_j [128 x 32] with all activation limbs [NA*TA x 32] at once and
// adds into TMEM columns [j*TA, (j+NA)*TA): column block b = i + j collects every limb product of weight 2^(8b).
// A decode batch of 1..16 rows therefore uses the same kernel with TA = 16.
//
// Warp roles (576 threads): warp 0 = TMA producer, warp 1 = TMEM allocation + MMA issue, warps 2..17 = epilogue:
// four groups of four warps; a warp may only access the 32 TMEM lanes of its warp id modulo 4, so the four warps of
// a group cover the 128 lanes and the groups share the accumulator columns (the epilogue is integer-ALU latency
// bound, one warp per scheduler would leave the ALUs idle). Stages of the shared-memory ring are handed over with
// mbarriers; every wait is bounded and a timeout ends the CTA with an error status instead of a hang.
#pragma once

#include "bx_ptx.cuh"

namespace bx {

constexpr int EPI_GROUPS = 4;
constexpr int GEMM_THREADS = 64 + 128 * EPI_GROUPS;
constexpr int WROWS = 128;   // weight rows per CTA (MMA M)
constexpr int BKB = 128;     // K bytes per stage (one 128-byte swizzle atom per row)
constexpr int UMMA_K = 32;   // int8 K per MMA


template <int NW, int NA, int TA>
struct GemmCfg {
  static_assert(TA % 16 == 0 && TA >= 16, "activation tile: multiple of 16 rows");
  static_assert(NA * TA <= 256, "MMA N limit");
  static constexpr int NBLK = NW + NA - 1;                  // accumulator column blocks
  static constexpr int COLS = NBLK * TA;                    // TMEM columns in use
  static constexpr int TMEM_COLS = COLS <= 32 ? 32 : COLS <= 64 ? 64 : COLS <= 128 ? 128 : COLS <= 256 ? 256 : 512;
  static_assert(COLS <= 512, "TMEM capacity");
  static constexpr int W_BYTES = NW * WROWS * BKB;
  static constexpr int A_BYTES = NA * TA * BKB;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  static constexpr int SMEM_BUDGET = 227 * 1024 - 2048;     // ring budget; the rest holds barriers + alignment slack
  static constexpr int STAGES_MAX = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_MAX > 6 ? 6 : STAGES_MAX;
  static_assert(STAGES >= 2, "at least two stages");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

struct GemmShared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// Runs the main loop for the output tile (weight rows n0.., activation rows m0..) over k blocks [kb0, kb1).
// On return, for warps 2..5, the accumulators are complete in TMEM (returns false after a timeout).
// Epi::run(tmem_base, lane_quarter, group, lane, ...) is called by the epilogue warps.
template <int NW, int NA, int TA, class Epi>
__device__ __forceinline__ void limb_gemm_tile(const CUtensorMap* tmap_w, const CUtensorMap* tmap_a, int n0, int m0,
                                               int kb0, int kb1, const typename Epi::Params& ep) {
  using Cfg = GemmCfg<NW, NA, TA>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmShared* sh = reinterpret_cast<GemmShared*>(ring + Cfg::STAGES * Cfg::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    mbar_init(&sh->acc_full, 1);
    // A timeout anywhere earlier (sticky until the host clears it) makes every later CTA leave at once.
    sh->abort_flag = *reinterpret_cast<volatile int*>(&g_wait_timeouts) != 0;
    fence_barrier_init();
    tma_prefetch_desc(tmap_w);
    tma_prefetch_desc(tmap_a);
  }
  __syncthreads();
  if (sh->abort_flag) return;
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
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
        tma_load_3d(st, tmap_w, &sh->full[s], (kb0 + i) * BKB, n0, 0);
        tma_load_3d(st + Cfg::W_BYTES, tmap_a, &sh->full[s], (kb0 + i) * BKB, m0, 0);
        issued = i + 1;
      }
      if (!ok) {
        atomicAdd(&g_wait_timeouts, 1);
        sh->abort_flag = 1;
        // let the copies already in flight land before the CTA can exit
        for (int i = (issued > Cfg::STAGES ? issued - Cfg::STAGES : 0); i < issued; ++i)
          mbar_wait(&sh->full[i % Cfg::STAGES], (i / Cfg::STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issue ----
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
            // First K slice: every column block is written exactly once without accumulation.
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
        umma_commit(&sh->empty[s]);        // stage free once these MMAs have read it
      }
      if (ok) {
        umma_commit(&sh->acc_full);
      } else {
        atomicAdd(&g_wait_timeouts, 1);
        sh->abort_flag = 1;
      }
    }
  } else {
    // ---- epilogue warps: row constants and L1 prefetches first, they overlap the main loop ----
    const typename Epi::Row row = Epi::load_row(warp & 3, (warp - 2) >> 2, lane, n0, m0, ep);
    Epi::prefetch(row, (warp - 2) >> 2, lane, m0, ep);
    bool ok = true;
    if (nkb > 0) ok = mbar_wait(&sh->acc_full, 0);
    ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag) == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      Epi::run(tmem, warp & 3, (warp - 2) >> 2, lane, n0, m0, nkb > 0, ep, row);
    } else if (lane == 0) {
      atomicAdd(&g_wait_timeouts, 1);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Persistent variant: one CTA per SM walks a list of output tiles; two TMEM accumulator buffers let the epilogue of
// tile i run while the MMAs of tile i + 1 fill the other buffer, and the TMA producer runs ahead across tile
// boundaries. Needs 2 * COLS <= 512 TMEM columns (exact mode: TA <= 48).
struct GemmSharedP {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// NBUF accumulator buffers in TMEM (2: the epilogue of a tile runs behind the MMAs of the next one; 1: tiles too wide
// for two buffers, the MMAs of the next tile wait until the epilogue has read the accumulators out, while the TMA
// warp already fills the ring for it). W_FASTEST: consecutive tiles walk the 128-row operand first.
template <int NW, int NA, int TA, class Epi, int NBUF = 2, bool W_FASTEST = false>
__device__ __forceinline__ void limb_gemm_persistent(const CUtensorMap* tmap_w, const CUtensorMap* tmap_a, int n_tiles,
                                                     int m_tiles, int nkb, const typename Epi::Params& ep) {
  using Cfg = GemmCfg<NW, NA, TA>;
  static_assert(NBUF == 1 || NBUF == 2, "one or two accumulator buffers");
  static_assert(NBUF * Cfg::COLS <= 512, "the accumulator buffers must fit in TMEM");
  constexpr int UCOLS = NBUF * Cfg::COLS;
  constexpr int TCOLS = UCOLS <= 64 ? 64 : UCOLS <= 128 ? 128 : UCOLS <= 256 ? 256 : 512;
  auto w_origin = [&](int tile) { return (W_FASTEST ? tile % n_tiles : tile / m_tiles) * WROWS; };
  auto a_origin = [&](int tile) { return (W_FASTEST ? tile / n_tiles : tile % m_tiles) * TA; };
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmSharedP* sh = reinterpret_cast<GemmSharedP*>(ring + Cfg::STAGES * Cfg::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total = n_tiles * m_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 4 * EPI_GROUPS);
    }
    sh->abort_flag = *reinterpret_cast<volatile int*>(&g_wait_timeouts) != 0;
    fence_barrier_init();
    tma_prefetch_desc(tmap_w);
    tma_prefetch_desc(tmap_a);
  }
  __syncthreads();
  if (sh->abort_flag) return;
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, TCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: one continuous stream of stages over all tiles of this CTA ----
      int it = 0;            // global stage counter
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int n0 = w_origin(tile), m0 = a_origin(tile);
        for (int i = 0; i < nkb && ok; ++i, ++it) {
          const int s = it % Cfg::STAGES, round = it / Cfg::STAGES;
          if (round > 0) ok = mbar_wait(&sh->empty[s], (round - 1) & 1);
          if (!ok) break;
          uint8_t* st = ring + s * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&sh->full[s], Cfg::STAGE_BYTES);
          tma_load_3d(st, tmap_w, &sh->full[s], i * BKB, n0, 0);
          tma_load_3d(st + Cfg::W_BYTES, tmap_a, &sh->full[s], i * BKB, m0, 0);
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
    if (lane == 0) {
      // ---- MMA issue ----
      constexpr uint32_t ID_ALL = umma_idesc_i8(NA * TA);
      constexpr uint32_t ID_ONE = umma_idesc_i8(TA);
      constexpr uint32_t ID_REST = umma_idesc_i8(NA > 1 ? (NA - 1) * TA : TA);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++tcount) {
        const int buf = tcount % NBUF, use = tcount / NBUF;
        if (use > 0) ok = mbar_wait(&sh->acc_empty[buf], (use - 1) & 1);   // epilogue has drained this buffer
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem + buf * Cfg::COLS;
        for (int i = 0; i < nkb && ok; ++i, ++it) {
          const int s = it % Cfg::STAGES;
          ok = mbar_wait(&sh->full[s], (it / Cfg::STAGES) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t wbase = smem_u32(ring + s * Cfg::STAGE_BYTES);
          const uint32_t abase = wbase + Cfg::W_BYTES;
#pragma unroll
          for (int ks = 0; ks < BKB / UMMA_K; ++ks) {
            const uint32_t koff = ks * UMMA_K;
            const uint64_t adesc = umma_desc_sw128(abase + koff);
            if (i == 0 && ks == 0) {
              umma_i8(acc, umma_desc_sw128(wbase + koff), adesc, ID_ALL, 0);
#pragma unroll
              for (int j = 1; j < NW; ++j) {
                const uint64_t wdesc = umma_desc_sw128(wbase + j * (WROWS * BKB) + koff);
                umma_i8(acc + (j + NA - 1) * TA, wdesc, umma_desc_sw128(abase + (NA - 1) * TA * BKB + koff), ID_ONE, 0);
                if (NA > 1) umma_i8(acc + j * TA, wdesc, adesc, ID_REST, 1);
              }
            } else {
#pragma unroll
              for (int j = 0; j < NW; ++j)
                umma_i8(acc + j * TA, umma_desc_sw128(wbase + j * (WROWS * BKB) + koff), adesc, ID_ALL, 1);
            }
          }
          umma_commit(&sh->empty[s]);
        }
        if (ok) umma_commit(&sh->acc_full[buf]);
      }
      if (!ok) {
        atomicAdd(&g_wait_timeouts, 1);
        sh->abort_flag = 1;
      }
    }
  } else {
    // ---- epilogue warps ----
    int tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++tcount) {
      const int buf = tcount % NBUF, use = tcount / NBUF;
      const int n0 = w_origin(tile), m0 = a_origin(tile);
      // row constants and L1 prefetches before the wait: they overlap the MMAs of this tile
      const typename Epi::Row row = Epi::load_row(warp & 3, (warp - 2) >> 2, lane, n0, m0, ep);
      Epi::prefetch(row, (warp - 2) >> 2, lane, m0, ep);
      if (ok) ok = mbar_wait(&sh->acc_full[buf], use & 1);
      ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag) == 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if constexpr (NBUF == 1) {
        // One buffer: read the accumulators out into registers, hand the buffer back to the MMA warp at once, and do
        // the arithmetic and the stores behind the MMAs of the next tile.
        typename Epi::Drained acc;
        Epi::drain(tmem, warp & 3, (warp - 2) >> 2, lane, n0, m0, nkb > 0, ep, acc);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->acc_empty[0]);
        Epi::finish(acc, warp & 3, (warp - 2) >> 2, lane, n0, m0, ep, row);
      } else {
        Epi::run(tmem + buf * Cfg::COLS, warp & 3, (warp - 2) >> 2, lane, n0, m0, nkb > 0, ep, row);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->acc_empty[buf]);
      }
    }
    if (!ok && lane == 0) atomicAdd(&g_wait_timeouts, 1);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, TCOLS);
  }
}

}  // namespace bx
