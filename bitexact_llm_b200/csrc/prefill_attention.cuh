// Prefill attention over the paged int8 limb-plane KV cache: one CTA per tile of consecutive query tokens of one
// request and one KV head, both integer sweeps inside the CTA, the limb products on tcgen05.
//
// A tile is BT = 32 / G consecutive tokens x the G query heads of the KV head: 32 query rows r = t G + g, so a K / V
// row staged for the tile serves 32 queries (the per-row decode kernel stages it once per token). Same integers as
// the per-row kernel and as the reference's prefill kernel (src/bitexact/vllm_plugin/tri_prefill.py:32-86, int8
// weight rule) and, with the exact weight rule, as bmm + softmax_w + bmm (src/bitexact/exact/model.py:114-119):
// every product is an exact limb dot, the maximum and the sums are exact integer reductions, and key s is visible
// to a query iff s <= its position, so the grouping of queries into tiles cannot change a bit.
//
// Per block of 128 keys (staged by TMA, one box of 128 bytes x page rows per page and cache-row third:
// [K0|K1], [K2|V0], [V1|V2], 128-byte swizzle, no byte fetched twice):
//   scores  S^T [128 keys = TMEM lanes] x [5 blocks x 32 queries]: A = K limb j tile (K-major), B = the three
//           stacked query limb tiles [96 x 64] written once per tile; 8 MMAs; block b = i + j as in the limb GEMM.
//   sweep 1 keeps a running maximum per (thread, query row); sweep 2 recomputes the scores (the MMAs are a few
//           hundred cycles; keeping 32 x S int64 scores on chip is not possible), turns them into weights with the
//           final row maximum, and writes the weights' three limbs as the B operand [96 x 128 keys] of
//   p.V     D1 [lanes = bytes of [K2|V0]] and D2 [lanes = bytes of [V1|V2]] x [96 = (weight limb, query)], A = the
//           staged cache rows read MN-major (no transposition), accumulated in TMEM over ALL keys of the tile and
//           read once at the end (|sum| <= keys * 2^14 < 2^31 for fewer than 43690 keys).
// Thread layout: 16 warps; warp % 4 = TMEM lane quarter (32 keys), warp / 4 = group of 8 query rows.
// Every wait is bounded; a timeout ends the CTA with the device status word set.
#pragma once

#include "paged_attention.cuh"

namespace bx {

constexpr int PF_MAXROWS = 32;                  // query rows per tile: 32 (one CTA per SM) or 16 (two CTAs per SM)
constexpr int PF_KEYS = 128;                    // keys per block
constexpr int PF_BOX = PF_KEYS * 128;           // one third of the cache rows of a block: 16 KB
constexpr int PF_STAGE = 3 * PF_BOX;

// Sizes that follow from the tile height ROWS (3 ROWS limb rows in the query and weight tiles).
template <int ROWS>
struct PfCfg {
  static_assert(ROWS == 16 || ROWS == 32, "tile height");
  static constexpr int THREADS = 16 * ROWS;               // 4 lane quarters x ROWS / 8 row groups, one warp each
  static constexpr int RG = 3 * ROWS / 8;                 // 8-row groups of the limb tiles
  static constexpr int LBO = RG * 128;                    // bytes between the 16-byte K chunks of those tiles
  static constexpr int QTILE = 4 * LBO;                   // query limbs [3 ROWS x 64 dims] as 8 x 16-byte core matrices
  static constexpr int PTILE = 8 * LBO;                   // weight limbs [3 ROWS x 128 keys]
  static constexpr int S_COLS = 5 * ROWS;                 // score accumulators
  static constexpr int D1 = S_COLS, D2 = D1 + 3 * ROWS;   // p.V accumulators (3 ROWS columns each)
  static constexpr int TMEM = ROWS == 32 ? 512 : 256;
};

struct PrefillParams {
  const int32_t* q;     // [N, HKV, G, 64]
  const i64* sh;        // [N, HKV, G] (exact mode; null with ptab)
  const i64* pos;       // [N] query position of each token
  const int32_t* tiles; // [T, 3] (block-table row, first token, tokens <= 32 / G)
  const void* bt;
  int bt64;
  int64_t sbt;
  int nblk, bs;
  AttnParams w;         // weight rule: lut / l2e (exact) or ptab (int8)
  i64* num;             // [N, HKV, G, 64]
  i64* den;             // [N, HKV, G]
  int HKV, G;
};

struct PrefillSmall {
  uint64_t full[2];
  uint64_t mma_done;
  uint64_t pv_done;
  uint32_t tmem_base;
  uint32_t fail;
  i64 red[4][PF_MAXROWS];
};

template <int ROWS>
__global__ void __launch_bounds__(PfCfg<ROWS>::THREADS, ROWS == 32 ? 1 : 2)
prefill_attention_kernel(const __grid_constant__ CUtensorMap tmap, const PrefillParams p) {
  using C = PfCfg<ROWS>;
  constexpr int PF_ROWS = ROWS, PF_THREADS = C::THREADS, PF_LBO = C::LBO, PF_D1 = C::D1, PF_D2 = C::D2;
  extern __shared__ uint8_t pf_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_smem) + 1023) & ~uintptr_t(1023));
  uint8_t* qtile = ring + 2 * PF_STAGE;
  uint8_t* ptile = qtile + C::QTILE;
  PrefillSmall* sm = reinterpret_cast<PrefillSmall*>(ptile + C::PTILE);
  i64* comb = reinterpret_cast<i64*>(ring);            // after the last MMA: [32 rows][64 dims]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, group = warp >> 2;
  const int h = blockIdx.y;
  const int G = p.G;
  const int64_t brow = p.tiles[3 * blockIdx.x];
  const int64_t tok0 = p.tiles[3 * blockIdx.x + 1];
  const int ntok = p.tiles[3 * blockIdx.x + 2];

  if (tid == 0) {
    mbar_init(&sm->full[0], 1);
    mbar_init(&sm->full[1], 1);
    mbar_init(&sm->mma_done, 1);
    mbar_init(&sm->pv_done, 1);
    sm->fail = *reinterpret_cast<volatile int*>(&g_wait_timeouts) != 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 0) {
    tmem_alloc(&sm->tmem_base, C::TMEM);
    tmem_relinquish();
  }
  // ---- the three query limb tiles: row (i, r) of the B operand, 16-byte K chunks PF_LBO apart ----
  for (int e = tid; e < PF_ROWS * 16; e += PF_THREADS) {       // 4 consecutive dims per step
    const int r = e >> 4, d0 = (e & 15) * 4;
    const int t = r / G, g = r % G;
    int4 v = make_int4(0, 0, 0, 0);
    if (t < ntok) v = *reinterpret_cast<const int4*>(p.q + (((tok0 + t) * p.HKV + h) * G + g) * ATT_HD + d0);
    int x[4] = {v.x, v.y, v.z, v.w};
    uint32_t w[3] = {0, 0, 0};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int i = 0; i < 3; ++i) w[i] |= (uint32_t)(split8(x[c]) & 255) << (8 * c);
    }
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int row = i * PF_ROWS + r;
      *reinterpret_cast<uint32_t*>(qtile + (d0 >> 4) * PF_LBO + (row >> 3) * 128 + (row & 7) * 16 + (d0 & 15)) = w[i];
    }
  }
  // this thread's 8 query rows
  int qp[8];
  i64 rshift[8];
  i64 kmax = -1;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r = 8 * group + j, t = r / G;
    qp[j] = -1;
    rshift[j] = 0;
    if (t < ntok) {
      const i64 pq = p.pos[tok0 + t];
      qp[j] = (int)imin(pq, (i64)p.nblk * p.bs - 1);
      if (p.sh) rshift[j] = (i64)(FK + 3 - FZ) - p.sh[((tok0 + t) * p.HKV + h) * G + (r % G)];
    }
  }
  for (int t = 0; t < ntok; ++t) kmax = imax(kmax, imin(p.pos[tok0 + t], (i64)p.nblk * p.bs - 1));
  const int kend = (int)(kmax + 1);
  const int nb = (kend + PF_KEYS - 1) / PF_KEYS;
  const int pages = PF_KEYS / p.bs;                    // pages per block
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
  bool failed = sm->fail != 0;

  // ---- producer: one block of keys into stage it % 2 (sweep 1 needs only the K thirds) ----
  auto load = [&](int it) {
    const int sweep = it / nb, blk = it % nb, st = it & 1;
    uint8_t* base = ring + st * PF_STAGE;
    mbar_arrive_expect_tx(&sm->full[st], (sweep ? 3 : 2) * PF_BOX);
    for (int pg = 0; pg < pages; ++pg) {
      const int pidx = blk * pages + pg;
      int64_t b = 0;                                   // pages past the table: the null block (its keys are masked)
      if (pidx < p.nblk)
        b = p.bt64 ? reinterpret_cast<const int64_t*>(p.bt)[brow * p.sbt + pidx]
                   : (int64_t) reinterpret_cast<const int32_t*>(p.bt)[brow * p.sbt + pidx];
      const int off = pg * p.bs * 128;
      tma_load_4d(base + off, &tmap, &sm->full[st], 0, 0, h, (int)b);
      tma_load_4d(base + PF_BOX + off, &tmap, &sm->full[st], 128, 0, h, (int)b);
      if (sweep) tma_load_4d(base + 2 * PF_BOX + off, &tmap, &sm->full[st], 256, 0, h, (int)b);
    }
  };

  i64 mx[8], den[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    mx[j] = ATT_NEG;
    den[j] = 0;
  }
  const int total = 2 * nb;
  int issued = 0;
  if (!failed && nb > 0) {
    if (tid == 0) load(0);
    issued = 1;
  }
  constexpr uint32_t ID_ALL = umma_idesc_i8(3 * PF_ROWS), ID_ONE = umma_idesc_i8(PF_ROWS), ID_TWO = umma_idesc_i8(2 * PF_ROWS);
  constexpr uint32_t ID_PV = umma_idesc_i8_amn(3 * PF_ROWS);
  const uint32_t qaddr = smem_u32(qtile), paddr = smem_u32(ptile);

  for (int it = 0; it < total && !failed; ++it) {
    const int sweep = it / nb, blk = it % nb, st = it & 1;
    if (it + 1 < total) {
      if (tid == 0) load(it + 1);                      // the other stage: its last readers finished an iteration ago
      issued = it + 2;
    }
    bool ok = mbar_wait(&sm->full[st], (it >> 1) & 1);
    const uint32_t sbase = smem_u32(ring + st * PF_STAGE);
    if (ok && tid == 0) {
      // ---- scores of the block: 8 MMAs ----
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const uint32_t qk = qaddr + ks * 2 * PF_LBO;
        const uint64_t q_all = umma_desc_kmajor_plain(qk, PF_LBO, 128);
        const uint64_t k0 = umma_desc_sw128(sbase + ks * 32), k1 = umma_desc_sw128(sbase + 64 + ks * 32);
        const uint64_t k2 = umma_desc_sw128(sbase + PF_BOX + ks * 32);
        if (ks == 0) {
          // every column block written once without accumulation
          const uint64_t q_two = q_all, q_last = umma_desc_kmajor_plain(qk + (2 * PF_ROWS / 8) * 128, PF_LBO, 128);
          umma_i8(tmem, k0, q_all, ID_ALL, 0);
          umma_i8(tmem + 3 * PF_ROWS, k1, q_last, ID_ONE, 0);
          umma_i8(tmem + 1 * PF_ROWS, k1, q_two, ID_TWO, 1);
          umma_i8(tmem + 4 * PF_ROWS, k2, q_last, ID_ONE, 0);
          umma_i8(tmem + 2 * PF_ROWS, k2, q_two, ID_TWO, 1);
        } else {
          umma_i8(tmem, k0, q_all, ID_ALL, 1);
          umma_i8(tmem + 1 * PF_ROWS, k1, q_all, ID_ALL, 1);
          umma_i8(tmem + 2 * PF_ROWS, k2, q_all, ID_ALL, 1);
        }
      }
      umma_commit(&sm->mma_done);
    }
    ok = ok && mbar_wait(&sm->mma_done, it & 1);
    if (__syncthreads_or(!ok)) {
      failed = true;
      break;
    }
    tc_fence_after();
    // ---- this thread: key lane of the block, 8 query rows ----
    const int key = blk * PF_KEYS + quarter * 32 + lane;
    uint32_t acc[5][8];
#pragma unroll
    for (int b = 0; b < 5; ++b) tmem_ld8(tmem + lane_base + b * PF_ROWS + 8 * group, acc[b]);
    tmem_ld_wait();
    i64 raw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      raw[j] = (i64)(int32_t)acc[0][j] + shl((i64)(int32_t)acc[1][j], 8) + shl((i64)(int32_t)acc[2][j], 16) +
               shl((i64)(int32_t)acc[3][j], 24) + shl((i64)(int32_t)acc[4][j], 32);
    if (sweep == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (key <= qp[j]) mx[j] = imax(mx[j], raw[j]);
      if (blk == nb - 1) {
        // ---- row maxima over all keys: lanes, then the four quarters ----
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          i64 v = mx[j];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = imax(v, __shfl_xor_sync(0xffffffffu, v, o));
          if (lane == 0) sm->red[quarter][8 * group + j] = v;
        }
      }
    } else {
      // ---- weights with the final maxima; their limbs are the B operand of p.V ----
      uint8_t* pcol = ptile + quarter * 2 * PF_LBO + (lane >> 4) * PF_LBO + group * 128 + (lane & 15);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        i64 pv = 0;
        if (key <= qp[j]) pv = attn_weight_any(p.w, raw[j], mx[j], rshift[j]);
        den[j] += pv;
        int rem = (int)pv;
#pragma unroll
        for (int i = 0; i < 3; ++i) pcol[i * (PF_ROWS / 8) * 128 + j * 16] = (uint8_t)split8(rem);
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();                                   // score accumulators read; weights written
    if (sweep == 0) {
      if (blk == nb - 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = 8 * group + j;
          mx[j] = imax(imax(sm->red[0][r], sm->red[1][r]), imax(sm->red[2][r], sm->red[3][r]));
        }
      }
    } else {
      bool okv = true;
      if (tid == 0) {
        tc_fence_after();
#pragma unroll
        for (int kg = 0; kg < 4; ++kg) {
          const uint64_t pdesc = umma_desc_kmajor_plain(paddr + kg * 2 * PF_LBO, PF_LBO, 128);
          const uint32_t accum = (blk > 0 || kg > 0) ? 1u : 0u;
          umma_i8(tmem + PF_D1, umma_desc_sw128(sbase + PF_BOX + kg * 4096), pdesc, ID_PV, accum);
          umma_i8(tmem + PF_D2, umma_desc_sw128(sbase + 2 * PF_BOX + kg * 4096), pdesc, ID_PV, accum);
        }
        umma_commit(&sm->pv_done);
      }
      okv = mbar_wait(&sm->pv_done, blk & 1);          // the weight tile and the stage are free again
      if (__syncthreads_or(!okv)) {
        failed = true;
        break;
      }
    }
  }

  if (failed) {
    if (tid == 0) {
      atomicAdd(&g_wait_timeouts, 1);
      // let the copies in flight land before the CTA can exit
      for (int i = (issued > 2 ? issued - 2 : 0); i < issued; ++i) mbar_wait(&sm->full[i & 1], (i >> 1) & 1);
    }
  } else if (nb > 0) {
    // ---- sums of the weights: lanes, then quarters ----
    tc_fence_after();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      i64 v = den[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) sm->red[quarter][8 * group + j] = v;
    }
    // ---- p.V accumulators: lane = byte of the cache-row third, column 32 i + r = (weight limb i, query r) ----
    uint32_t d1[3][8], d2[3][8];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      tmem_ld8(tmem + lane_base + PF_D1 + i * PF_ROWS + 8 * group, d1[i]);
      tmem_ld8(tmem + lane_base + PF_D2 + i * PF_ROWS + 8 * group, d2[i]);
    }
    tmem_ld_wait();
    i64 part[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      i64 a = 0;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        // quarters 0, 1: D2 lanes = V limb 1; quarters 2, 3: D1 lanes = V limb 0, D2 lanes = V limb 2
        const i64 v = quarter < 2 ? shl((i64)(int32_t)d2[i][j], 8)
                                  : (i64)(int32_t)d1[i][j] + shl((i64)(int32_t)d2[i][j], 16);
        a += shl(v, 8 * i);
      }
      part[j] = a;
    }
    __syncthreads();                                   // every MMA is complete (pv_done of the last block): ring is free
    const int d = (quarter & 1) * 32 + lane;
    if (quarter < 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) comb[(8 * group + j) * ATT_HD + d] = part[j];
    }
    __syncthreads();
    if (quarter >= 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = 8 * group + j, t = r / G;
        if (t < ntok)
          p.num[(((tok0 + t) * p.HKV + h) * G + (r % G)) * ATT_HD + d] = part[j] + comb[r * ATT_HD + d];
      }
    }
    if (tid < PF_ROWS) {
      const int r = tid, t = r / G;
      if (t < ntok)
        p.den[((tok0 + t) * p.HKV + h) * G + (r % G)] = sm->red[0][r] + sm->red[1][r] + sm->red[2][r] + sm->red[3][r];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM);
  }
}

}  // namespace bx
