// Exact-mode integer attention over the paged int8 limb-plane KV cache, for M <= 4 query rows per (request,
// KV head): the G query heads of one decode token, or one prefill token.
//
//   raw[i, s] = sum_d q[i, d] K[s, d]                 exact (int8 limb products, int32 partials, int64 join)
//   mx[i]     = max over s <= qpos[i] of raw[i, s]
//   p[i, s]   = 2^-t at 22 bits, t from (mx - raw) by the row-shift / log2(e) / table + interpolation rule
//   den[i]    = sum_s p,  num[i, d] = sum_s p V[s, d]  exact int64
//
// The weights need the FINAL row maximum (the quantised table does not satisfy exp(a) exp(b) = exp(a + b)), so the
// keys are swept twice. Here the first sweep keeps the exact scores in shared memory and the second sweep never
// touches K again: each key's 384 cache bytes are read from HBM exactly once. A (request, head) pair is split
// over a thread-block CLUSTER: each CTA owns a contiguous key range, the row maxima and the partial sums are
// exchanged through distributed shared memory; no atomics, no zero fills, no second kernel.
//
// Same integers as tri_exact_attn.attend (src/bitexact/vllm_plugin/tri_exact_attn.py:67-165) and as the unfused
// bmm + softmax_w + bmm of src/bitexact/exact/model.py:114-119: all reductions are exact integer sums / maxima.
// Cache row (512 bytes per block, head, slot): K limbs at [0, 192), V limbs at [192, 384)
// (src/bitexact/vllm_plugin/tri_paged.py:22-25).
#pragma once

#include <cooperative_groups.h>

#include "bx_ptx.cuh"
#include "bx_rules.cuh"

namespace bx {

namespace cg = cooperative_groups;

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int ATT_HD = 64;
constexpr int ATT_MAXCS = 8;
constexpr i64 ATT_NEG = -(1ll << 62);
constexpr i64 ZMAX = 48ll << FZ;

struct AttnParams {
  const int32_t* q;     // [R, HKV, M, 64]
  const i64* sh;        // [R, HKV, M]
  const i64* qpos;      // [R, M]
  const int8_t* cache;  // [nb, HKV, bs, 512]
  int64_t sc_nb, sc_h, sc_bs;
  int bs;
  const void* bt;       // block table [*, nblk], int32 or int64
  int bt64;
  int64_t sbt;
  int nblk;
  const i64* rmap;      // [R] block-table row of each q row (null: identity)
  const i64* lut;       // 2^-f table, 16385 entries at 2^60
  i64 l2e;
  i64* num;             // [R, HKV, M, 64]
  i64* den;             // [R, HKV, M]
  int M, HKV;
  int chunk_cap;        // score slots per query row in shared memory (multiple of 8)
  const int32_t* ptab;  // int8 mode: weight table rsh(e^z table, 10), 131073 entries; null = exact mode
};

struct AttnShared {
  i64 pnum[ATT_WARPS][4][ATT_HD];
  i64 cnum[4][ATT_HD];
  i64 pden[ATT_WARPS][4];
  i64 cden[4];
  i64 wmax[ATT_WARPS][4];
  i64 cmax[4];
  int pw[ATT_WARPS][8][4];
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ i64 attn_weight(i64 raw, i64 mx, i64 rowshift, i64 l2e, const i64* __restrict__ lut) {
  const i64 z = mx - raw;
  const i64 zf = imin(rshc(z, rowshift), ZMAX);
  const i64 t = (zf * l2e + (1ll << (FZ + 28 - FT2 - 1))) >> (FZ + 28 - FT2);
  const i64 n = t >> FT2;
  const i64 f = t & ((1ll << FT2) - 1);
  const int idx = (int)(f >> (FT2 - EXP2_BITS));
  const i64 rr = f & ((1ll << (FT2 - EXP2_BITS)) - 1);
  const i64 a = __ldg(lut + idx);
  const i64 b = __ldg(lut + idx + 1);
  const i64 v = a + rshs<FT2 - EXP2_BITS>((b - a) * rr);
  const int s = (int)imin((i64)(EXP2_ONE - FP) + n, 62);
  return (v + (1ll << (s - 1))) >> s;
}

// The weight of one (query, key) pair in either mode. int8 mode (src/bitexact/int8/segs.py:91-99, fused copy
// src/bitexact/vllm_plugin/tri_paged.py:171-175, head_dim 64): z = rsh(raw - mx, 2*14 + 3 - 12), direct table
// lookup, 0 below the table.
__device__ __forceinline__ i64 attn_weight_any(const AttnParams& p, i64 raw, i64 mx, i64 rowshift) {
  if (p.ptab) {
    constexpr int ZSH = 2 * 14 + 3 - 12;
    constexpr i64 ZLO = -(32ll << 12);
    const i64 z = ((raw - mx) + (1ll << (ZSH - 1))) >> ZSH;
    const i64 idx = imax(z, ZLO - 1) - ZLO;
    return idx >= 0 ? (i64)__ldg(p.ptab + idx) : 0;
  }
  return attn_weight(raw, mx, rowshift, p.l2e, p.lut);
}

__global__ void __launch_bounds__(ATT_THREADS)
exact_attention_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t att_smem[];
  AttnShared* sm = reinterpret_cast<AttnShared*>(att_smem);
  i64* scores = reinterpret_cast<i64*>(att_smem + sizeof(AttnShared));     // [4][chunk_cap]

  cg::cluster_group cluster = cg::this_cluster();
  const int CS = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int64_t pz = blockIdx.x / CS;            // (request, KV head); the cluster lies along x
  const int64_t r = pz / p.HKV;
  const int h = (int)(pz % p.HKV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Key range of this CTA.
  i64 kend = 0;
  for (int g = 0; g < p.M; ++g) kend = imax(kend, p.qpos[r * p.M + g] + 1);
  kend = imin(kend, (i64)p.nblk * p.bs);
  const i64 per = (kend + CS - 1) / CS;
  i64 chunk = (per + 7) / 8 * 8;
  if (chunk > p.chunk_cap) chunk = p.chunk_cap;   // cannot happen for kend <= nblk * bs; keeps indices in range
  const i64 lo = imin((i64)rank * chunk, kend);
  const i64 hi = imin(lo + chunk, kend);
  const i64 brow = p.rmap ? p.rmap[r] : r;
  const int8_t* cbase = p.cache + (int64_t)h * p.sc_h;

  auto key_offset = [&](i64 key) -> int64_t {     // byte offset of the key's cache row (key < hi)
    const i64 bi = key / p.bs;
    const i64 blk = p.bt64 ? reinterpret_cast<const i64*>(p.bt)[brow * p.sbt + bi]
                           : (i64) reinterpret_cast<const int32_t*>(p.bt)[brow * p.sbt + bi];
    return blk * p.sc_nb + (key % p.bs) * p.sc_bs;
  };

  // ---- A fragments: the 3 limbs of the M query rows stacked as 16 MMA rows (limb i of query g at row 4 i + g) ----
  uint32_t afrag[2][4];
  {
    const int row_lo = lane >> 2;
    const int g = row_lo & 3;
    const int limb_lo = row_lo >> 2;                        // 0 or 1
    const bool hi_used = row_lo < 4;                        // rows 8..11 = limb 2
    const int32_t* qrow = p.q + (pz * p.M + g) * ATT_HD;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int d0 = 32 * t + 16 * half + (lane & 3) * 4;
        uint32_t wl = 0, wh = 0;
        if (g < p.M) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            int v = qrow[d0 + b];
            const int l0 = split8(v), l1 = split8(v), l2 = split8(v);
            wl |= (uint32_t)((limb_lo ? l1 : l0) & 255) << (8 * b);
            wh |= (uint32_t)(l2 & 255) << (8 * b);
          }
        }
        afrag[t][2 * half] = wl;
        afrag[t][2 * half + 1] = hi_used ? wh : 0u;
      }
    }
  }

  // ---- sweep 1: exact scores into shared memory, row maxima ----
  i64 mymax[2] = {ATT_NEG, ATT_NEG};                        // lanes 0..15: query g = lane / 4
  const i64 qp_s1 = (lane < 16 && (lane >> 2) < p.M) ? p.qpos[r * p.M + (lane >> 2)] : -1;
  for (i64 kb = lo + 8 * warp; kb < hi; kb += 8 * ATT_WARPS) {
    const i64 key = kb + (lane >> 2);
    int acc[3][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
    uint32_t bfrag[3][2][2];
    if (key < hi) {
      const int8_t* kp = cbase + key_offset(key) + (lane & 3) * 4;
#pragma unroll
      for (int j = 0; j < 3; ++j)
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          bfrag[j][t][0] = *reinterpret_cast<const uint32_t*>(kp + j * ATT_HD + 32 * t);
          bfrag[j][t][1] = *reinterpret_cast<const uint32_t*>(kp + j * ATT_HD + 32 * t + 16);
        }
    } else {
#pragma unroll
      for (int j = 0; j < 3; ++j)
#pragma unroll
        for (int t = 0; t < 2; ++t) bfrag[j][t][0] = bfrag[j][t][1] = 0u;
    }
#pragma unroll
    for (int j = 0; j < 3; ++j)
#pragma unroll
      for (int t = 0; t < 2; ++t) mma_s8(acc[j], afrag[t], bfrag[j][t][0], bfrag[j][t][1]);
    // join the K limbs; the row's own limb weight is applied below
    i64 slo[2], shi[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      slo[c] = (i64)acc[0][c] + shl((i64)acc[1][c], 8) + shl((i64)acc[2][c], 16);
      shi[c] = (i64)acc[0][2 + c] + shl((i64)acc[1][2 + c], 8) + shl((i64)acc[2][2 + c], 16);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const i64 mid = __shfl_down_sync(0xffffffffu, slo[c], 16);      // limb 1 of the same query and key
      if (lane < 16) {
        const i64 raw = slo[c] + shl(mid, 8) + shl(shi[c], 16);
        const i64 kk = kb + (lane & 3) * 2 + c;
        const int g = lane >> 2;
        if (kk < hi) {
          scores[(int64_t)g * p.chunk_cap + (kk - lo)] = raw;
          if (kk <= qp_s1) mymax[c] = imax(mymax[c], raw);
        }
      }
    }
  }
  {
    i64 m = imax(mymax[0], mymax[1]);
    m = imax(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = imax(m, __shfl_xor_sync(0xffffffffu, m, 2));
    if (lane < 16 && (lane & 3) == 0) sm->wmax[warp][lane >> 2] = m;
  }
  __syncthreads();
  if (threadIdx.x < 4) {
    i64 m = ATT_NEG;
    for (int w = 0; w < ATT_WARPS; ++w) m = imax(m, sm->wmax[w][threadIdx.x]);
    sm->cmax[threadIdx.x] = m;
  }
  cluster.sync();

  // ---- sweep 2: weights from the global maxima, den and num = p V ----
  const int g2 = lane & 3;
  i64 mx = ATT_NEG;
  for (int c = 0; c < CS; ++c) mx = imax(mx, cluster.map_shared_rank(sm->cmax, c)[g2]);
  const bool gok = g2 < p.M;
  const i64 qp2 = gok ? p.qpos[r * p.M + g2] : -1;
  const i64 rowshift = (gok && p.sh) ? (i64)(FK + 3 - FZ) - p.sh[pz * p.M + g2] : 0;
  i64 den = 0;
  i64 nacc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) nacc[a][b] = 0;
  const int half = lane >> 4, dg = lane & 15;
  for (i64 kb = lo + 8 * warp; kb < hi; kb += 8 * ATT_WARPS) {
    const i64 mykey = kb + (lane >> 2);
    i64 pv = 0;
    if (mykey < hi && mykey <= qp2) pv = attn_weight_any(p, scores[(int64_t)g2 * p.chunk_cap + (mykey - lo)], mx, rowshift);
    den += pv;
    const i64 kfor = kb + (lane & 7);
    const int64_t off = kfor < hi ? key_offset(kfor) : 0;
    __syncwarp();
    sm->pw[warp][lane >> 2][g2] = (int)pv;
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int kk = 2 * it + half;
      const int64_t voff = __shfl_sync(0xffffffffu, off, kk);
      if (kb + kk < hi) {
        const int8_t* vp = cbase + voff + 3 * ATT_HD + 4 * dg;
        const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vp);
        const uint32_t w1 = *reinterpret_cast<const uint32_t*>(vp + ATT_HD);
        const uint32_t w2 = *reinterpret_cast<const uint32_t*>(vp + 2 * ATT_HD);
        const int4 pq = *reinterpret_cast<const int4*>(&sm->pw[warp][kk][0]);
        const int pg[4] = {pq.x, pq.y, pq.z, pq.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int v = (int)(int8_t)(w0 >> (8 * c)) + ((int)(int8_t)(w1 >> (8 * c)) << 8) +
                        ((int)(int8_t)(w2 >> (8 * c)) << 16);
#pragma unroll
          for (int a = 0; a < 4; ++a) nacc[a][c] += (i64)pg[a] * (i64)v;
        }
      }
    }
  }
  // combine the two key parities, then warps, then the cluster
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      nacc[a][c] += __shfl_xor_sync(0xffffffffu, nacc[a][c], 16);
      if (lane < 16) sm->pnum[warp][a][4 * dg + c] = nacc[a][c];
    }
  den += __shfl_xor_sync(0xffffffffu, den, 4);
  den += __shfl_xor_sync(0xffffffffu, den, 8);
  den += __shfl_xor_sync(0xffffffffu, den, 16);
  if (lane < 4) sm->pden[warp][lane] = den;
  __syncthreads();
  {
    const int g = threadIdx.x >> 6, d = threadIdx.x & 63;
    i64 s = 0;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) s += sm->pnum[w][g][d];
    sm->cnum[g][d] = s;
    if (threadIdx.x < 4) {
      i64 t = 0;
      for (int w = 0; w < ATT_WARPS; ++w) t += sm->pden[w][threadIdx.x];
      sm->cden[threadIdx.x] = t;
    }
  }
  cluster.sync();
  if (rank == 0) {
    const int g = threadIdx.x >> 6, d = threadIdx.x & 63;
    if (g < p.M) {
      i64 s = 0;
      for (int c = 0; c < CS; ++c) s += cluster.map_shared_rank(&sm->cnum[0][0], c)[g * ATT_HD + d];
      p.num[(pz * p.M + g) * ATT_HD + d] = s;
    }
    if (threadIdx.x < p.M) {
      i64 t = 0;
      for (int c = 0; c < CS; ++c) t += cluster.map_shared_rank(sm->cden, c)[threadIdx.x];
      p.den[pz * p.M + threadIdx.x] = t;
    }
  }
  cluster.sync();                                   // remote shared memory stays valid until rank 0 has read it
}

}  // namespace bx

// =====================================================================================================================
// TMA-staged variant (page sizes 8, 16, 32, 64; 16-byte aligned cache strides). Same integers, same cluster layout.
//
// A producer warp streams the cache pages of the CTA's key range through a shared-memory ring with
// cp.async.bulk.tensor (4-D map over the cache: byte, slot, head, block; box = 192 bytes x page): first the K halves
// of the rows (sweep 1), then the V halves (sweep 2), 64 keys per stage. Eight consumer warps take 8 keys of every
// stage each: q.K with mma.sync from shared-memory fragments (one 16-byte load per limb), exact scores into
// shared memory, then weights and p.V from the staged V rows. Hand-over by full / empty mbarriers with bounded waits.
namespace bx {

constexpr int ATT2_STAGE_KEYS = 64;
constexpr int ATT2_HALF = 192;                                  // bytes of K (or V) limbs per cache row
constexpr int ATT2_STAGE_BYTES = ATT2_STAGE_KEYS * ATT2_HALF;   // 12288
constexpr int ATT2_NS = 4;
constexpr int ATT2_THREADS = ATT_THREADS + 32;                  // 8 consumer warps + 1 producer warp

struct Attn2Small {
  i64 cnum[4][ATT_HD];
  i64 pden[ATT_WARPS][4];
  i64 cden[4];
  i64 wmax[ATT_WARPS][4];
  i64 cmax[4];
  int pw[ATT_WARPS][8][4];
  uint64_t full[ATT2_NS];
  uint64_t empty[ATT2_NS];
  uint32_t abort_flag;
};

__global__ void __launch_bounds__(ATT2_THREADS, 2)
exact_attention_tma_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p) {
  extern __shared__ __align__(128) uint8_t att_smem[];
  uint8_t* ring = att_smem;                                                        // [NS][64 keys][192 B]
  i64* scores = reinterpret_cast<i64*>(att_smem + ATT2_NS * ATT2_STAGE_BYTES);     // [chunk_cap][4]
  Attn2Small* sm = reinterpret_cast<Attn2Small*>(att_smem + ATT2_NS * ATT2_STAGE_BYTES + (size_t)p.chunk_cap * 32);
  i64 (*pnum)[4][ATT_HD] = reinterpret_cast<i64 (*)[4][ATT_HD]>(ring);             // aliases the ring after the sweeps

  cg::cluster_group cluster = cg::this_cluster();
  const int CS = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int64_t pz = blockIdx.x / CS;
  const int64_t r = pz / p.HKV;
  const int h = (int)(pz % p.HKV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  i64 kend = 0;
  for (int g = 0; g < p.M; ++g) kend = imax(kend, p.qpos[r * p.M + g] + 1);
  kend = imin(kend, (i64)p.nblk * p.bs);
  const i64 per = (kend + CS - 1) / CS;
  i64 chunk = (per + ATT2_STAGE_KEYS - 1) / ATT2_STAGE_KEYS * ATT2_STAGE_KEYS;
  if (chunk > p.chunk_cap) chunk = p.chunk_cap;
  const i64 lo = imin((i64)rank * chunk, kend);
  const i64 hi = imin(lo + chunk, kend);
  const int nst = (int)((hi - lo + ATT2_STAGE_KEYS - 1) / ATT2_STAGE_KEYS);
  const i64 brow = p.rmap ? p.rmap[r] : r;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ATT2_NS; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], ATT_WARPS);
    }
    sm->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap);
  }
  __syncthreads();

  if (warp == ATT_WARPS) {
    // ---------------- producer warp ----------------
    const int pages_per_stage = ATT2_STAGE_KEYS / p.bs;
    bool ok = true;
    for (int idx = 0; idx < 2 * nst; ++idx) {
      if (idx == nst) cluster_arrive();                            // sweep-1 loads are all issued
      const int sweep = idx >= nst, st = idx - sweep * nst;
      const int slot = idx % ATT2_NS, round = idx / ATT2_NS;
      if (ok && round > 0) ok = mbar_wait(&sm->empty[slot], (round - 1) & 1);
      if (!ok) continue;                                           // keep the barrier protocol, load nothing more
      const i64 key0 = lo + (i64)st * ATT2_STAGE_KEYS;
      int npages = (int)((hi - key0 + p.bs - 1) / p.bs);
      if (npages > pages_per_stage) npages = pages_per_stage;
      if (lane == 0) mbar_arrive_expect_tx(&sm->full[slot], (uint32_t)(npages * p.bs * ATT2_HALF));
      __syncwarp();
      if (lane < npages) {
        const i64 bi = key0 / p.bs + lane;
        const i64 blk = p.bt64 ? reinterpret_cast<const i64*>(p.bt)[brow * p.sbt + bi]
                               : (i64) reinterpret_cast<const int32_t*>(p.bt)[brow * p.sbt + bi];
        tma_load_4d(ring + slot * ATT2_STAGE_BYTES + lane * p.bs * ATT2_HALF, &tmap, &sm->full[slot],
                    sweep ? ATT2_HALF : 0, 0, h, (int)blk);
      }
    }
    if (nst == 0) cluster_arrive();
    if (!ok && lane == 0) { atomicAdd(&g_wait_timeouts, 1); sm->abort_flag = 1; }
    cluster_wait();
    cluster.sync();
    cluster.sync();
    return;
  }

  // ---------------- consumer warps ----------------
  // A fragments: limb i of query g at MMA row 4 i + g; contraction slot (t, half, byte b) of lane c holds
  // dim 16 c + 4 (2 t + half) + b, which matches one 16-byte shared-memory load per K limb on the B side.
  uint32_t afrag[2][4];
  {
    const int row_lo = lane >> 2;
    const int g = row_lo & 3;
    const int limb_lo = row_lo >> 2;
    const bool hi_used = row_lo < 4;
    const int32_t* qrow = p.q + (pz * p.M + g) * ATT_HD;
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int d0 = 16 * (lane & 3) + 4 * (2 * t + half);
        uint32_t wl = 0, wh = 0;
        if (g < p.M) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            int v = qrow[d0 + b];
            const int l0 = split8(v), l1 = split8(v), l2 = split8(v);
            wl |= (uint32_t)((limb_lo ? l1 : l0) & 255) << (8 * b);
            wh |= (uint32_t)(l2 & 255) << (8 * b);
          }
        }
        afrag[t][2 * half] = wl;
        afrag[t][2 * half + 1] = hi_used ? wh : 0u;
      }
  }

  bool ok = true;
  // ---- sweep 1 ----
  i64 mymax[2] = {ATT_NEG, ATT_NEG};
  const i64 qp_s1 = (lane < 16 && (lane >> 2) < p.M) ? p.qpos[r * p.M + (lane >> 2)] : -1;
  for (int st = 0; st < nst; ++st) {
    const int slot = st % ATT2_NS, round = st / ATT2_NS;
    if (ok) ok = mbar_wait(&sm->full[slot], round & 1);
    ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sm->abort_flag) == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const i64 kb = lo + (i64)st * ATT2_STAGE_KEYS + 8 * warp;
      if (kb < hi) {
        const uint8_t* kp = ring + slot * ATT2_STAGE_BYTES + (8 * warp + (lane >> 2)) * ATT2_HALF + 16 * (lane & 3);
        int acc[3][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
        const bool kvalid = kb + (lane >> 2) < hi;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          uint4 w = make_uint4(0, 0, 0, 0);
          if (kvalid) w = *reinterpret_cast<const uint4*>(kp + j * ATT_HD);
          mma_s8(acc[j], afrag[0], w.x, w.y);
          mma_s8(acc[j], afrag[1], w.z, w.w);
        }
        i64 slo[2], shi[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          slo[c] = (i64)acc[0][c] + shl((i64)acc[1][c], 8) + shl((i64)acc[2][c], 16);
          shi[c] = (i64)acc[0][2 + c] + shl((i64)acc[1][2 + c], 8) + shl((i64)acc[2][2 + c], 16);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const i64 mid = __shfl_down_sync(0xffffffffu, slo[c], 16);
          if (lane < 16) {
            const i64 raw = slo[c] + shl(mid, 8) + shl(shi[c], 16);
            const i64 kk = kb + (lane & 3) * 2 + c;
            if (kk < hi) {
              scores[(kk - lo) * 4 + (lane >> 2)] = raw;
              if (kk <= qp_s1) mymax[c] = imax(mymax[c], raw);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->empty[slot]);
  }
  {
    i64 m = imax(mymax[0], mymax[1]);
    m = imax(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = imax(m, __shfl_xor_sync(0xffffffffu, m, 2));
    if (lane < 16 && (lane & 3) == 0) sm->wmax[warp][lane >> 2] = m;
  }
  asm volatile("bar.sync 1, %0;" ::"r"(ATT_THREADS) : "memory");        // the 8 consumer warps only
  if (threadIdx.x < 4) {
    i64 m = ATT_NEG;
    for (int w = 0; w < ATT_WARPS; ++w) m = imax(m, sm->wmax[w][threadIdx.x]);
    sm->cmax[threadIdx.x] = m;
  }
  cluster.sync();

  // ---- sweep 2 ----
  const int g2 = lane & 3;
  i64 mx = ATT_NEG;
  for (int c = 0; c < CS; ++c) mx = imax(mx, cluster.map_shared_rank(sm->cmax, c)[g2]);
  const bool gok = g2 < p.M;
  const i64 qp2 = gok ? p.qpos[r * p.M + g2] : -1;
  const i64 rowshift = (gok && p.sh) ? (i64)(FK + 3 - FZ) - p.sh[pz * p.M + g2] : 0;
  i64 den = 0;
  i64 nacc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) nacc[a][b] = 0;
  const int half = lane >> 4, dg = lane & 15;
  for (int st = 0; st < nst; ++st) {
    const int idx = nst + st;
    const int slot = idx % ATT2_NS, round = idx / ATT2_NS;
    if (ok) ok = mbar_wait(&sm->full[slot], round & 1);
    ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sm->abort_flag) == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const i64 kb = lo + (i64)st * ATT2_STAGE_KEYS + 8 * warp;
      if (kb < hi) {
        const i64 mykey = kb + (lane >> 2);
        i64 pv = 0;
        if (mykey < hi && mykey <= qp2) pv = attn_weight_any(p, scores[(mykey - lo) * 4 + g2], mx, rowshift);
        den += pv;
        sm->pw[warp][lane >> 2][g2] = (int)pv;
        __syncwarp();
        const uint8_t* vbase = ring + slot * ATT2_STAGE_BYTES + (8 * warp) * ATT2_HALF + 4 * dg;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int kk = 2 * it + half;
          if (kb + kk < hi) {
            const uint8_t* vp = vbase + kk * ATT2_HALF;
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vp);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(vp + ATT_HD);
            const uint32_t w2 = *reinterpret_cast<const uint32_t*>(vp + 2 * ATT_HD);
            const int4 pq = *reinterpret_cast<const int4*>(&sm->pw[warp][kk][0]);
            const int pg[4] = {pq.x, pq.y, pq.z, pq.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int v = (int)(int8_t)(w0 >> (8 * c)) + ((int)(int8_t)(w1 >> (8 * c)) << 8) +
                            ((int)(int8_t)(w2 >> (8 * c)) << 16);
#pragma unroll
              for (int a = 0; a < 4; ++a) nacc[a][c] += (i64)pg[a] * (i64)v;
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->empty[slot]);
  }
  if (!ok && lane == 0) atomicAdd(&g_wait_timeouts, 1);
  asm volatile("bar.sync 1, %0;" ::"r"(ATT_THREADS) : "memory");        // every stage is consumed: the ring is free
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      nacc[a][c] += __shfl_xor_sync(0xffffffffu, nacc[a][c], 16);
      if (lane < 16) pnum[warp][a][4 * dg + c] = nacc[a][c];
    }
  den += __shfl_xor_sync(0xffffffffu, den, 4);
  den += __shfl_xor_sync(0xffffffffu, den, 8);
  den += __shfl_xor_sync(0xffffffffu, den, 16);
  if (lane < 4) sm->pden[warp][lane] = den;
  asm volatile("bar.sync 1, %0;" ::"r"(ATT_THREADS) : "memory");
  {
    const int g = threadIdx.x >> 6, d = threadIdx.x & 63;
    i64 s = 0;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) s += pnum[w][g][d];
    sm->cnum[g][d] = s;
    if (threadIdx.x < 4) {
      i64 t = 0;
      for (int w = 0; w < ATT_WARPS; ++w) t += sm->pden[w][threadIdx.x];
      sm->cden[threadIdx.x] = t;
    }
  }
  cluster.sync();
  if (rank == 0) {
    const int g = threadIdx.x >> 6, d = threadIdx.x & 63;
    if (g < p.M) {
      i64 s = 0;
      for (int c = 0; c < CS; ++c) s += cluster.map_shared_rank(&sm->cnum[0][0], c)[g * ATT_HD + d];
      p.num[(pz * p.M + g) * ATT_HD + d] = s;
    }
    if (threadIdx.x < p.M) {
      i64 t = 0;
      for (int c = 0; c < CS; ++c) t += cluster.map_shared_rank(sm->cden, c)[threadIdx.x];
      p.den[pz * p.M + threadIdx.x] = t;
    }
  }
  cluster.sync();
}

}  // namespace bx

// =====================================================================================================================
// Tensor-memory variant: as the TMA-staged kernel, but p.V runs on tcgen05 with the accumulators in TMEM.
//
// The contraction of p.V is over KEYS, while the cache rows hold DIMS contiguously. tcgen05 reads an "MN-major"
// int8 operand directly from shared memory, so the staged V rows need no transposition: the A operand is the V tile
// [32 keys x 128 bytes] (bytes = limb 0 | limb 1 of the 64 dims; a second tile holds limb 1 | limb 2, so that no byte outside the limbs is
// fetched: its limb 1 half is computed twice and ignored), loaded by TMA with the
// 128-byte swizzle; the B operand is the tile of p limbs [16 rows = (limb i, query g)] x [32 keys], K-major, written
// by the consumer warps. D [128 lanes = (V limb, dim)] x [16 columns = (p limb, query)] accumulates in TMEM over
// ALL keys of the CTA (|sum| <= keys * 2^14 < 2^31) and is read once at the end, so the per-key work of sweep 2
// is only the weight function and three byte stores.
namespace bx {

constexpr int ATT3_STAGE_BYTES = ATT2_STAGE_KEYS * 256;        // 16384: [V0|V1] tile 8 KB + [V1|V2] tile 8 KB
#ifndef BX_ATT3_NS
#define BX_ATT3_NS 3
#endif
constexpr int ATT3_NS = BX_ATT3_NS;
constexpr int ATT3_TMEM_COLS = 32;

struct Attn3Small {
  i64 cnum[4][ATT_HD];
  i64 pden[ATT_WARPS][4];
  i64 cden[4];
  i64 wmax[ATT_WARPS][4];
  i64 cmax[4];
  uint64_t full[ATT3_NS];
  uint64_t empty_k[ATT3_NS];     // sweep 1: the 8 consumer warps release a stage
  uint64_t empty_v[ATT3_NS];     // sweep 2: tcgen05.commit releases a stage
  uint64_t acc_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// K-major, unswizzled operand tile: 8-row core matrices of 16 bytes per row; lbo = bytes between the two 16-byte K
// chunks, sbo = bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_kmajor_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// int8 x int8 -> int32, A MN-major, B K-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc_i8_amn(int n) {
  return umma_idesc_i8(n) | (1u << 15);
}

// NW consumer warps (4 or 8) take 8 keys of every stage each: a stage is 8 NW keys. Smaller CTAs (NW = 4) put more
// independent load streams on an SM.
template <int NW>
__global__ void __launch_bounds__(32 * NW + 32, NW == 4 ? 5 : 3)
exact_attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                          const AttnParams p) {
  constexpr int KEYS = 8 * NW;                  // keys per stage
  constexpr int STAGE_BYTES = KEYS * 256;       // [V0|V1] tile + [V1|V2] tile (the K half uses 192 B per key)
  constexpr int CTHREADS = 32 * NW;             // consumer threads
  extern __shared__ __align__(128) uint8_t att_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_smem) + 1023) & ~uintptr_t(1023));
  i64* scores = reinterpret_cast<i64*>(ring + ATT3_NS * STAGE_BYTES);   // later, in place: the p-limb tiles
  Attn3Small* sm = reinterpret_cast<Attn3Small*>(reinterpret_cast<uint8_t*>(scores) + (size_t)p.chunk_cap * 32);

  cg::cluster_group cluster = cg::this_cluster();
  const int CS = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int64_t pz = blockIdx.x / CS;
  const int64_t r = pz / p.HKV;
  const int h = (int)(pz % p.HKV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  i64 kend = 0;
  for (int g = 0; g < p.M; ++g) kend = imax(kend, p.qpos[r * p.M + g] + 1);
  kend = imin(kend, (i64)p.nblk * p.bs);
  const i64 per = (kend + CS - 1) / CS;
  i64 chunk = (per + KEYS - 1) / KEYS * KEYS;
  if (chunk > p.chunk_cap) chunk = p.chunk_cap;
  const i64 lo = imin((i64)rank * chunk, kend);
  const i64 hi = imin(lo + chunk, kend);
  const int nst = (int)((hi - lo + KEYS - 1) / KEYS);
  const i64 brow = p.rmap ? p.rmap[r] : r;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ATT3_NS; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty_k[s], NW);
      mbar_init(&sm->empty_v[s], 1);
    }
    mbar_init(&sm->acc_done, 1);
    sm->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 0) {
    tmem_alloc(&sm->tmem_base, ATT3_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;

  if (warp == NW) {
    // ---------------- producer warp ----------------
    // Block-table entries are fetched 32 pages at a time (one per lane) and handed out by shuffles, so that issuing a
    // stage never waits for a global load.
    const int pages_per_stage = KEYS / p.bs;
    const i64 pg0 = lo / p.bs;
    const int npg = (int)((hi - lo + p.bs - 1) / p.bs);
    auto load_bt = [&](int block) -> i64 {
      const int rel = block * 32 + lane;
      if (rel >= npg) return 0;
      return p.bt64 ? reinterpret_cast<const i64*>(p.bt)[brow * p.sbt + pg0 + rel]
                    : (i64) reinterpret_cast<const int32_t*>(p.bt)[brow * p.sbt + pg0 + rel];
    };
    int cur_block = 0;
    i64 my_bt = load_bt(0);
    bool ok = true;
    for (int idx = 0; idx < 2 * nst; ++idx) {
      if (idx == nst) cluster_arrive();
      const int sweep = idx >= nst, st = idx - sweep * nst;
      const int slot = idx % ATT3_NS;
      const int rel0 = st * pages_per_stage;                        // first page of the stage (a stage never straddles
      if (rel0 / 32 != cur_block) {                                 // a block of 32 pages: pages_per_stage divides 32)
        cur_block = rel0 / 32;
        my_bt = load_bt(cur_block);
      }
      const i64 blk = __shfl_sync(0xffffffffu, my_bt, (rel0 + lane) & 31);
      const int prev = idx - ATT3_NS;                               // previous use of this slot
      if (ok && prev >= 0) {
        if (prev < nst) {
          ok = mbar_wait(&sm->empty_k[slot], (prev / ATT3_NS) & 1);
        } else {                                                    // ordinal of `prev` among this slot's sweep-2 uses
          const int ord = (prev + ATT3_NS - 1 - slot) / ATT3_NS - (nst + ATT3_NS - 1 - slot) / ATT3_NS;
          ok = mbar_wait(&sm->empty_v[slot], ord & 1);
        }
      }
      if (!ok) continue;
      const i64 key0 = lo + (i64)st * KEYS;
      int npages = (int)((hi - key0 + p.bs - 1) / p.bs);
      if (npages > pages_per_stage) npages = pages_per_stage;
      if (lane == 0)
        mbar_arrive_expect_tx(&sm->full[slot], (uint32_t)(npages * p.bs * (sweep ? 256 : ATT2_HALF)));
      __syncwarp();
      if (lane < npages) {
        uint8_t* st_base = ring + slot * STAGE_BYTES;
        if (!sweep) {
          tma_load_4d(st_base + lane * p.bs * ATT2_HALF, &tmap_k, &sm->full[slot], 0, 0, h, (int)blk);
        } else {
          tma_load_4d(st_base + lane * p.bs * 128, &tmap_v, &sm->full[slot], 192, 0, h, (int)blk);
          tma_load_4d(st_base + KEYS * 128 + lane * p.bs * 128, &tmap_v, &sm->full[slot], 256, 0, h, (int)blk);
        }
      }
    }
    if (nst == 0) cluster_arrive();
    if (!ok && lane == 0) { atomicAdd(&g_wait_timeouts, 1); sm->abort_flag = 1; }
    cluster_wait();
    cluster.sync();
    cluster.sync();
    __syncthreads();                                               // TMEM release point of the CTA
    return;
  }

  // ---------------- consumer warps ----------------
  uint32_t afrag[2][4];
  {
    const int row_lo = lane >> 2;
    const int g = row_lo & 3;
    const int limb_lo = row_lo >> 2;
    const bool hi_used = row_lo < 4;
    const int32_t* qrow = p.q + (pz * p.M + g) * ATT_HD;
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int d0 = 16 * (lane & 3) + 4 * (2 * t + half);
        uint32_t wl = 0, wh = 0;
        if (g < p.M) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            int v = qrow[d0 + b];
            const int l0 = split8(v), l1 = split8(v), l2 = split8(v);
            wl |= (uint32_t)((limb_lo ? l1 : l0) & 255) << (8 * b);
            wh |= (uint32_t)(l2 & 255) << (8 * b);
          }
        }
        afrag[t][2 * half] = wl;
        afrag[t][2 * half + 1] = hi_used ? wh : 0u;
      }
  }

  bool ok = true;
  // ---- sweep 1: scores (as the TMA-staged kernel) ----
  i64 mymax[2] = {ATT_NEG, ATT_NEG};
  const i64 qp_s1 = (lane < 16 && (lane >> 2) < p.M) ? p.qpos[r * p.M + (lane >> 2)] : -1;
  for (int st = 0; st < nst; ++st) {
    const int slot = st % ATT3_NS, round = st / ATT3_NS;
    if (ok) ok = mbar_wait(&sm->full[slot], round & 1);
    ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sm->abort_flag) == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const i64 kb = lo + (i64)st * KEYS + 8 * warp;
      if (kb < hi) {
        const uint8_t* kp = ring + slot * STAGE_BYTES + (8 * warp + (lane >> 2)) * ATT2_HALF + 16 * (lane & 3);
        int acc[3][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
        const bool kvalid = kb + (lane >> 2) < hi;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          uint4 w = make_uint4(0, 0, 0, 0);
          if (kvalid) w = *reinterpret_cast<const uint4*>(kp + j * ATT_HD);
          mma_s8(acc[j], afrag[0], w.x, w.y);
          mma_s8(acc[j], afrag[1], w.z, w.w);
        }
        i64 slo[2], shi[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          slo[c] = (i64)acc[0][c] + shl((i64)acc[1][c], 8) + shl((i64)acc[2][c], 16);
          shi[c] = (i64)acc[0][2 + c] + shl((i64)acc[1][2 + c], 8) + shl((i64)acc[2][2 + c], 16);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const i64 mid = __shfl_down_sync(0xffffffffu, slo[c], 16);
          if (lane < 16) {
            const i64 raw = slo[c] + shl(mid, 8) + shl(shi[c], 16);
            const i64 kk = kb + (lane & 3) * 2 + c;
            if (kk < hi) {
              scores[(kk - lo) * 4 + (lane >> 2)] = raw;
              if (kk <= qp_s1) mymax[c] = imax(mymax[c], raw);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->empty_k[slot]);
  }
  {
    i64 m = imax(mymax[0], mymax[1]);
    m = imax(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = imax(m, __shfl_xor_sync(0xffffffffu, m, 2));
    if (lane < 16 && (lane & 3) == 0) sm->wmax[warp][lane >> 2] = m;
  }
  asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");
  if (threadIdx.x < 4) {
    i64 m = ATT_NEG;
    for (int w = 0; w < NW; ++w) m = imax(m, sm->wmax[w][threadIdx.x]);
    sm->cmax[threadIdx.x] = m;
  }
  cluster.sync();

  // ---- sweep 2, phase A: weights of every key of this CTA, written in place of the scores as p-limb tiles ----
  // A group of 32 keys owns 1024 bytes of the score buffer; one warp reads its 128 scores (4 per lane), then
  // overwrites the first 512 bytes with the K-major tile [16 rows (limb, query)] x [32 keys].
  const int g2 = lane & 3;
  i64 mx = ATT_NEG;
  for (int c = 0; c < CS; ++c) mx = imax(mx, cluster.map_shared_rank(sm->cmax, c)[g2]);
  const bool gok = g2 < p.M;
  const i64 qp2 = gok ? p.qpos[r * p.M + g2] : -1;
  const i64 rowshift = (gok && p.sh) ? (i64)(FK + 3 - FZ) - p.sh[pz * p.M + g2] : 0;
  i64 den = 0;
  const int ngroups = (int)((hi - lo + 31) / 32);
  for (int grp = warp; grp < ngroups; grp += NW) {
    i64 sc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) sc[j] = scores[((i64)grp * 32 + 8 * j + (lane >> 2)) * 4 + g2];
    __syncwarp();
    uint8_t* pt = reinterpret_cast<uint8_t*>(scores) + (size_t)grp * 1024;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kl = 8 * j + (lane >> 2);
      const i64 key = lo + (i64)grp * 32 + kl;
      i64 pv = 0;
      if (key < hi && key <= qp2) pv = attn_weight_any(p, sc[j], mx, rowshift);
      den += pv;
      int pr = (int)pv;
      const int off = (kl >> 4) * 256 + (kl & 15) + g2 * 16;
      pt[off] = (uint8_t)split8(pr);                                // row g      (limb 0)
      pt[off + 64] = (uint8_t)split8(pr);                           // row 4 + g  (limb 1)
      pt[off + 128] = (uint8_t)split8(pr);                          // row 8 + g  (limb 2)
    }
  }
  fence_proxy_async_smem();
  asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");

  // ---- sweep 2, phase B: one thread streams the staged V tiles through tcgen05 ----
  constexpr uint32_t IDESC = umma_idesc_i8_amn(16);
  if (threadIdx.x == 0) {
    for (int st = 0; st < nst; ++st) {
      const int idx = nst + st;
      const int slot = idx % ATT3_NS, round = idx / ATT3_NS;
      if (ok) ok = mbar_wait(&sm->full[slot], round & 1);
      ok = ok && (*reinterpret_cast<volatile uint32_t*>(&sm->abort_flag) == 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t vbase = smem_u32(ring + slot * STAGE_BYTES);
#pragma unroll
      for (int kg = 0; kg < KEYS / 32; ++kg) {
        const int grp = (KEYS / 32) * st + kg;
        if (grp < ngroups) {
          const uint64_t bdesc = umma_desc_kmajor_plain(smem_u32(scores) + grp * 1024, 256, 128);
          const uint32_t accum = grp > 0 ? 1u : 0u;
          umma_i8(tmem, umma_desc_sw128(vbase + kg * 4096), bdesc, IDESC, accum);
          umma_i8(tmem + 16, umma_desc_sw128(vbase + KEYS * 128 + kg * 4096), bdesc, IDESC, accum);
        }
      }
      umma_commit(&sm->empty_v[slot]);
      if (st == nst - 1) umma_commit(&sm->acc_done);
    }
    if (!ok) { atomicAdd(&g_wait_timeouts, 1); sm->abort_flag = 1; }
  }
  __syncwarp();

  den += __shfl_xor_sync(0xffffffffu, den, 4);
  den += __shfl_xor_sync(0xffffffffu, den, 8);
  den += __shfl_xor_sync(0xffffffffu, den, 16);
  if (lane < 4) sm->pden[warp][lane] = den;

  // ---- read the accumulators: first tile lanes 0..63 = (V limb 0, dim), 64..127 = (V limb 1, dim); second tile
  //      lanes 64..127 = (V limb 2, dim) (its lanes 0..63 repeat limb 1 and are ignored).
  //      Column 4 i + g = (p limb i, query g). ----
  i64 part[4] = {0, 0, 0, 0};
  if (warp < 4) {
    bool done = ok && nst > 0;
    if (done) done = mbar_wait(&sm->acc_done, 0);
    done = done && (*reinterpret_cast<volatile uint32_t*>(&sm->abort_flag) == 0);
    done = __all_sync(0xffffffffu, done);
    if (done) {
      tc_fence_after();
      uint32_t d01[16], d12[16];
      const uint32_t tb = tmem + ((uint32_t)(warp * 32) << 16);
      tmem_ld16(tb, d01);
      tmem_ld16(tb + 16, d12);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        i64 a = (i64)(int32_t)d01[g] + shl((i64)(int32_t)d01[4 + g], 8) + shl((i64)(int32_t)d01[8 + g], 16);
        if (warp >= 2) {
          const i64 b = (i64)(int32_t)d12[g] + shl((i64)(int32_t)d12[4 + g], 8) + shl((i64)(int32_t)d12[8 + g], 16);
          a = shl(a, 8) + shl(b, 16);
        }
        part[g] = a;
      }
    }
  }
  tc_fence_before();
  asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");
  if (warp < 2) {
#pragma unroll
    for (int g = 0; g < 4; ++g) sm->cnum[g][warp * 32 + lane] = part[g];
  }
  asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");
  if (warp >= 2 && warp < 4) {
#pragma unroll
    for (int g = 0; g < 4; ++g) sm->cnum[g][(warp - 2) * 32 + lane] += part[g];
  }
  if (threadIdx.x < 4) {
    i64 t = 0;
    for (int w = 0; w < NW; ++w) t += sm->pden[w][threadIdx.x];
    sm->cden[threadIdx.x] = t;
  }
  cluster.sync();
  if (rank == 0) {
    for (int t = threadIdx.x; t < 4 * ATT_HD; t += CTHREADS) {
      const int g = t >> 6, d = t & 63;
      if (g < p.M) {
        i64 s = 0;
        for (int c = 0; c < CS; ++c) s += cluster.map_shared_rank(&sm->cnum[0][0], c)[g * ATT_HD + d];
        p.num[(pz * p.M + g) * ATT_HD + d] = s;
      }
    }
    if (threadIdx.x < p.M) {
      i64 t = 0;
      for (int c = 0; c < CS; ++c) t += cluster.map_shared_rank(sm->cden, c)[threadIdx.x];
      p.den[pz * p.M + threadIdx.x] = t;
    }
  }
  cluster.sync();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, ATT3_TMEM_COLS);
  }
}

}  // namespace bx

// =====================================================================================================================
// Persistent streaming variant for decode batches with many (request, KV head) pairs and contexts whose scores fit in
// shared memory: no clusters; every CTA walks a list of pairs and its producer warp keeps the ring of TMA stages
// full ACROSS pair boundaries (K stages of a pair, its V stages, K stages of the next pair, ...), so the HBM stream
// of an SM does not stop while the consumer warps run the phases that read no new bytes (row maxima, weight pass,
// accumulator read-out). One ring and one pair of barriers per slot serve both sweeps: a K stage is released by the
// NW consumer warps, a V stage by the tcgen05.commit of its MMAs plus NW - 1 arrivals of the issuing thread.
// A separate warp issues the MMAs: it takes a 32-key group as soon as the group's weights are written (a tagged flag
// per group, release / acquire), so V stages drain while the rest of the weight pass is still running.
// Pairs are dealt round robin (pair = block index + k * grid size): handing them out through a global ticket counter
// was measured and lost more to the extra hand-over per pair than it gained on ragged batches. With up to 512
// requests every CTA first ranks the requests by context length (longest first, ties by index: the same order in
// every CTA), so that the round robin hands every CTA a like mix of long and short pairs.
//
// Long contexts: a pair whose scores do not fit the shared-memory buffer (C keys) keeps them in a per-CTA slice of a
// caller-provided scratch buffer instead (written in sweep 1, read back once by the weight pass: 64 extra bytes per
// key, mostly L2 traffic), and sweep 2 runs in chunks of C keys: the weights of a chunk are written as p-limb tiles
// into the shared-memory buffer, the MMA warp consumes the chunk's V stages, and the buffer is reused for the next
// chunk once the chunk's MMAs have completed (acc_done is committed per chunk). One CTA therefore owns a pair of
// any length, with no cluster and no cross-CTA exchange, and the CTAs stay small enough for three or four per SM.
//
// V tiles: [V limb 0 | V limb 1] (cache bytes 192..319) and [V limb 1 | V limb 2] (bytes 256..383), both 128-byte
// swizzled rows, so no byte outside the limbs is fetched; TMEM lanes 0..63 of the second accumulator repeat limb 1
// and are ignored. The arithmetic is that of the kernel above.
namespace bx {

constexpr int ATT6_MAXNS = 8;
constexpr int ATT6_MAXGROUPS = 160;        // 32-key groups per pair (5120 keys)

struct Attn6Small {
  i64 cnum[4][ATT_HD];
  i64 pden[ATT_WARPS][4];
  i64 wmax[ATT_WARPS][4];
  uint64_t full[ATT6_MAXNS];
  uint64_t empty[ATT6_MAXNS];
  uint64_t acc_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t ptag[ATT6_MAXGROUPS];           // ordinal + 1 of the pair whose weights the group's p tile holds
};

__device__ __forceinline__ void flag_release(uint32_t* f, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(f)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t flag_acquire(const uint32_t* f) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(f)) : "memory");
  return v;
}
// Bounded wait for *f == want.
__device__ __forceinline__ bool flag_wait(const uint32_t* f, uint32_t want) {
  if (flag_acquire(f) == want) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (flag_acquire(f) == want) return true;
    if (clock64() - t0 > BX_WAIT_CYCLES) return false;
  }
}

template <int NW>
__global__ void __launch_bounds__(32 * NW + 64, NW == 4 ? 4 : 2)
exact_attention_stream_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                              const AttnParams p, int NS, int64_t npairs, i64* spill, int64_t spill_keys) {
  constexpr int KEYS = 8 * NW;                  // keys per stage
  constexpr int STAGE_BYTES = KEYS * 256;       // two V tiles of 128-byte rows (the K sweep uses 192 B per key)
  constexpr int CTHREADS = 32 * NW;             // consumer threads
  extern __shared__ __align__(128) uint8_t att_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_smem) + 1023) & ~uintptr_t(1023));
  i64* scores = reinterpret_cast<i64*>(ring + (size_t)NS * STAGE_BYTES);   // later, in place: the p-limb tiles
  Attn6Small* sm = reinterpret_cast<Attn6Small*>(reinterpret_cast<uint8_t*>(scores) + (size_t)p.chunk_cap * 32);
  uint16_t* order = reinterpret_cast<uint16_t*>(sm + 1);             // requests, longest context first (or unused)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C = p.chunk_cap;                                          // keys whose scores / p tiles fit in shared memory
  const int GPC = C / 32;                                             // 32-key groups per chunk (a multiple of NW)
  i64* my_spill = spill ? spill + (size_t)blockIdx.x * spill_keys * 4 : nullptr;
  const int64_t nreq = npairs / p.HKV;
  bool ranked = nreq <= 512 && C >= 128;                              // the sort's tables borrow the score buffer

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], NW);
    }
    mbar_init(&sm->acc_done, 1);
    sm->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  for (int i = threadIdx.x; i < ATT6_MAXGROUPS; i += blockDim.x) sm->ptag[i] = 0;
  if (ranked) {
    // Requests by context length, longest first, in buckets of 128 keys (ties by index): a counting sort whose
    // placement step runs in one warp over 32 requests at a time (match_any gives each lane its place among the lanes
    // of the same bucket), so every CTA computes the same order. The score buffer is still free: it holds the table.
    int* lens = reinterpret_cast<int*>(scores);                       // [512] bucket of each request
    int* base = lens + 512;                                           // [512] running start of each bucket
    for (int t = threadIdx.x; t < 512; t += blockDim.x) base[t] = 0;
    __syncthreads();
    for (int t = threadIdx.x; t < nreq; t += blockDim.x) {
      i64 kend = 0;
      for (int g = 0; g < p.M; ++g) kend = imax(kend, p.qpos[(int64_t)t * p.M + g] + 1);
      kend = imin(imax(kend, 0), (i64)p.nblk * p.bs);
      lens[t] = 511 - (int)imin(kend >> 7, 511);                       // bucket 0 = the longest contexts
    }
    __syncthreads();
    bool same = true;
    for (int t = threadIdx.x; t < nreq; t += blockDim.x) {
      const int b = lens[t];
      same &= b == lens[0];
      atomicAdd(&base[b], 1);
    }
    // every request in one bucket (a batch of like contexts): the given order is as good as any
    ranked = !__syncthreads_and(same);
    if (ranked && warp == 0) {
      // exclusive prefix of the 512 bucket counts: 16 per lane, then a warp scan
      int cnt[16], sum = 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) { cnt[i] = base[16 * lane + i]; sum += cnt[i]; }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int run = incl - sum;
#pragma unroll
      for (int i = 0; i < 16; ++i) { base[16 * lane + i] = run; run += cnt[i]; }
      __syncwarp();
      for (int t0 = 0; t0 < nreq; t0 += 32) {
        const int t = t0 + lane;
        const bool live = t < nreq;
        const int b = live ? lens[t] : -1 - lane;                     // dead lanes: buckets of their own
        const unsigned same = __match_any_sync(0xffffffffu, b);
        const int place = __popc(same & ((1u << lane) - 1));
        int start = 0;
        if (live) start = base[b];
        __syncwarp();
        if (live && place == 0) base[b] = start + __popc(same);
        __syncwarp();
        if (live) order[start + place] = (uint16_t)t;
      }
    }
  }
  if (warp == 0) {
    tmem_alloc(&sm->tmem_base, ATT3_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(&sm->abort_flag);
  constexpr uint32_t IDESC = umma_idesc_i8_amn(16);

  // the w-th piece of work: heads of the w / HKV-th longest request
  auto pair_of = [&](int64_t w) -> int64_t {
    if (!ranked) return w;
    return (int64_t)order[w / p.HKV] * p.HKV + w % p.HKV;
  };
  auto keys_of = [&](int64_t pz) -> i64 {
    const int64_t r = pz / p.HKV;
    i64 kend = 0;
    for (int g = 0; g < p.M; ++g) kend = imax(kend, p.qpos[r * p.M + g] + 1);
    kend = imin(kend, (i64)p.nblk * p.bs);
    return imin(kend, my_spill ? (i64)spill_keys : (i64)C);
  };

  if (warp == NW) {
    // ---------------- producer warp ----------------
    const int pages_per_stage = KEYS / p.bs;
    bool ok = true;
    uint32_t gidx = 0;                                               // stages issued so far, over all pairs
    for (int64_t w = blockIdx.x; w < npairs; w += gridDim.x) {
      const int64_t pz = pair_of(w);
      const int64_t r = pz / p.HKV;
      const int h = (int)(pz % p.HKV);
      const i64 hi = keys_of(pz);
      const int nst = (int)((hi + KEYS - 1) / KEYS);
      const i64 brow = p.rmap ? p.rmap[r] : r;
      const int npg = (int)((hi + p.bs - 1) / p.bs);
      // Block-table entries, 32 pages per fetch (one per lane), handed out by shuffles.
      auto load_bt = [&](int block) -> i64 {
        const int rel = block * 32 + lane;
        if (rel >= npg) return 0;
        return p.bt64 ? reinterpret_cast<const i64*>(p.bt)[brow * p.sbt + rel]
                      : (i64) reinterpret_cast<const int32_t*>(p.bt)[brow * p.sbt + rel];
      };
      int cur_block = 0;
      i64 my_bt = load_bt(0);
      for (int idx = 0; idx < 2 * nst; ++idx, ++gidx) {
        const int sweep = idx >= nst, st = idx - sweep * nst;
        const uint32_t slot = gidx % (uint32_t)NS, use = gidx / (uint32_t)NS;
        const int rel0 = st * pages_per_stage;                       // a stage never straddles a block of 32 pages
        if (rel0 / 32 != cur_block) {
          cur_block = rel0 / 32;
          my_bt = load_bt(cur_block);
        }
        const i64 blk = __shfl_sync(0xffffffffu, my_bt, (rel0 + lane) & 31);
        if (ok && use > 0) ok = mbar_wait(&sm->empty[slot], (use - 1) & 1);
        ok = ok && (*abort_flag == 0);
        if (!ok) continue;
        int npages = npg - rel0;
        if (npages > pages_per_stage) npages = pages_per_stage;
        if (lane == 0)
          mbar_arrive_expect_tx(&sm->full[slot], (uint32_t)(npages * p.bs * (sweep ? 256 : ATT2_HALF)));
        __syncwarp();
        if (lane < npages) {
          uint8_t* st_base = ring + (size_t)slot * STAGE_BYTES;
          if (!sweep) {
            tma_load_4d(st_base + lane * p.bs * ATT2_HALF, &tmap_k, &sm->full[slot], 0, 0, h, (int)blk);
          } else {
            tma_load_4d(st_base + lane * p.bs * 128, &tmap_v, &sm->full[slot], 192, 0, h, (int)blk);
            tma_load_4d(st_base + KEYS * 128 + lane * p.bs * 128, &tmap_v, &sm->full[slot], 256, 0, h, (int)blk);
          }
        }
      }
    }
    if (!ok && lane == 0) { atomicAdd(&g_wait_timeouts, 1); sm->abort_flag = 1; }
    __syncthreads();                                                 // TMEM release point of the CTA
    return;
  }

  if (warp == NW + 1) {
    // ---------------- MMA warp: one thread streams the staged V tiles through tcgen05 ----------------
    if (lane == 0) {
      bool ok = true;
      uint32_t gidx = 0, wave = 0;                                   // wave: chunks handed over so far, over all pairs
      constexpr int GPS = KEYS / 32;                                 // groups per stage
      for (int64_t w = blockIdx.x; w < npairs; w += gridDim.x) {
        const int64_t pz = pair_of(w);
        const i64 hi = keys_of(pz);
        const int nst = (int)((hi + KEYS - 1) / KEYS);
        const int ngroups = (int)((hi + 31) / 32);
        gidx += (uint32_t)nst;                                       // the K stages of the pair
        int ck = 0, cbase = 0;                                       // chunk of the stage's groups and its first group
        for (int st = 0; st < nst; ++st, ++gidx) {
          const uint32_t slot = gidx % (uint32_t)NS, use = gidx / (uint32_t)NS;
          const int g0 = GPS * st;                                   // first group of the stage
          if (g0 - cbase >= GPC) { ++ck; cbase += GPC; }             // (kept by counting: no division per stage)
          // The group's weights come first: they exist only after sweep 1 of this pair has consumed every K stage,
          // so the slot is at most one use behind and the parity wait below cannot mistake an older phase of the
          // barrier for this one.
          if (ok) ok = flag_wait(&sm->ptag[g0 - cbase], wave + ck + 1);
          if (ok) ok = mbar_wait(&sm->full[slot], use & 1);
          ok = ok && (*abort_flag == 0);
          if (!ok) continue;
          const uint32_t vbase = smem_u32(ring + (size_t)slot * STAGE_BYTES);
#pragma unroll
          for (int kg = 0; kg < GPS; ++kg) {
            const int grp = GPS * st + kg;
            const int place = grp - cbase;                           // GPC is a multiple of GPS: same chunk as g0
            if (grp < ngroups && ok) {
              if (kg > 0) ok = flag_wait(&sm->ptag[place], wave + ck + 1);
              if (ok) {
                tc_fence_after();
                const uint64_t bdesc = umma_desc_kmajor_plain(smem_u32(scores) + place * 1024, 256, 128);
                const uint32_t accum = grp > 0 ? 1u : 0u;
                umma_i8(tmem, umma_desc_sw128(vbase + kg * 4096), bdesc, IDESC, accum);
                umma_i8(tmem + 16, umma_desc_sw128(vbase + KEYS * 128 + kg * 4096), bdesc, IDESC, accum);
              }
            }
          }
          if (!ok) continue;
          umma_commit(&sm->empty[slot]);                             // one of the NW arrivals of the slot's phase
          for (int a = 1; a < NW; ++a) mbar_arrive(&sm->empty[slot]);
          // the chunk's last group (or the pair's): its p tiles may be overwritten, the accumulators read
          const int gend = GPS * (st + 1) < ngroups ? GPS * (st + 1) : ngroups;
          if (st == nst - 1 || gend - cbase == GPC) umma_commit(&sm->acc_done);
        }
        wave += (uint32_t)((ngroups + GPC - 1) / GPC);
      }
      if (!ok) { atomicAdd(&g_wait_timeouts, 1); sm->abort_flag = 1; }
    }
    __syncwarp();
    __syncthreads();                                                 // TMEM release point of the CTA
    return;
  }

  // ---------------- consumer warps ----------------
  bool ok = true;
  uint32_t gidx = 0;
  uint32_t wave = 0;                                                 // chunks handed over so far (acc_done phases)
  for (int64_t w = blockIdx.x; w < npairs; w += gridDim.x) {
    const int64_t pz = pair_of(w);
    const int64_t r = pz / p.HKV;
    const i64 hi = keys_of(pz);
    const int nst = (int)((hi + KEYS - 1) / KEYS);
    const bool spilled = hi > C;                                     // the scores of this pair live in the scratch slice

    uint32_t afrag[2][4];
    {
      const int row_lo = lane >> 2;
      const int g = row_lo & 3;
      const int limb_lo = row_lo >> 2;
      const bool hi_used = row_lo < 4;
      const int32_t* qrow = p.q + (pz * p.M + g) * ATT_HD;
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int d0 = 16 * (lane & 3) + 4 * (2 * t + half);
          uint32_t wl = 0, wh = 0;
          if (g < p.M) {
            const int4 qv = *reinterpret_cast<const int4*>(qrow + d0);
            const int qe[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              int v = qe[b];
              const int l0 = split8(v), l1 = split8(v), l2 = split8(v);
              wl |= (uint32_t)((limb_lo ? l1 : l0) & 255) << (8 * b);
              wh |= (uint32_t)(l2 & 255) << (8 * b);
            }
          }
          afrag[t][2 * half] = wl;
          afrag[t][2 * half + 1] = hi_used ? wh : 0u;
        }
    }

    // ---- sweep 1: scores ----
    i64 mymax[2] = {ATT_NEG, ATT_NEG};
    const i64 qp_s1 = (lane < 16 && (lane >> 2) < p.M) ? p.qpos[r * p.M + (lane >> 2)] : -1;
    for (int st = 0; st < nst; ++st, ++gidx) {
      const uint32_t slot = gidx % (uint32_t)NS, use = gidx / (uint32_t)NS;
      if (ok) ok = mbar_wait(&sm->full[slot], use & 1);
      ok = ok && (*abort_flag == 0);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        const i64 kb = (i64)st * KEYS + 8 * warp;
        if (kb < hi) {
          const uint8_t* kp = ring + (size_t)slot * STAGE_BYTES + (8 * warp + (lane >> 2)) * ATT2_HALF + 16 * (lane & 3);
          int acc[3][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
          const bool kvalid = kb + (lane >> 2) < hi;
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            uint4 w = make_uint4(0, 0, 0, 0);
            if (kvalid) w = *reinterpret_cast<const uint4*>(kp + j * ATT_HD);
            mma_s8(acc[j], afrag[0], w.x, w.y);
            mma_s8(acc[j], afrag[1], w.z, w.w);
          }
          i64 slo[2], shi[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            slo[c] = (i64)acc[0][c] + shl((i64)acc[1][c], 8) + shl((i64)acc[2][c], 16);
            shi[c] = (i64)acc[0][2 + c] + shl((i64)acc[1][2 + c], 8) + shl((i64)acc[2][2 + c], 16);
          }
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const i64 mid = __shfl_down_sync(0xffffffffu, slo[c], 16);
            if (lane < 16) {
              const i64 raw = slo[c] + shl(mid, 8) + shl(shi[c], 16);
              const i64 kk = kb + (lane & 3) * 2 + c;
              if (kk < hi) {
                if (spilled) my_spill[kk * 4 + (lane >> 2)] = raw;
                else scores[kk * 4 + (lane >> 2)] = raw;
                if (kk <= qp_s1) mymax[c] = imax(mymax[c], raw);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->empty[slot]);
    }
    {
      i64 m = imax(mymax[0], mymax[1]);
      m = imax(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = imax(m, __shfl_xor_sync(0xffffffffu, m, 2));
      if (lane < 16 && (lane & 3) == 0) sm->wmax[warp][lane >> 2] = m;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");

    // ---- sweep 2: weights, written in place of the scores as p-limb tiles (one warp per 32 keys) ----
    const int g2 = lane & 3;
    i64 mx = ATT_NEG;
#pragma unroll
    for (int w = 0; w < NW; ++w) mx = imax(mx, sm->wmax[w][g2]);
    const bool gok = g2 < p.M;
    const i64 qp2 = gok ? p.qpos[r * p.M + g2] : -1;
    const i64 rowshift = (gok && p.sh) ? (i64)(FK + 3 - FZ) - p.sh[pz * p.M + g2] : 0;
    i64 den = 0;
    const int ngroups = (int)((hi + 31) / 32);
    const int nchunks = (ngroups + GPC - 1) / GPC;
    for (int ck = 0; ck < nchunks; ++ck) {
      if (ck > 0) {
        // the p tiles of the previous chunk are still being read by its MMAs until they are committed
        if (ok) ok = mbar_wait(&sm->acc_done, (wave + ck - 1) & 1);
        ok = ok && (*abort_flag == 0);
        ok = __all_sync(0xffffffffu, ok);
      }
      const int gtop = (ck + 1) * GPC < ngroups ? (ck + 1) * GPC : ngroups;
      for (int grp = ck * GPC + warp; grp < gtop; grp += NW) {
        const int place = grp - ck * GPC;
        i64 sc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const i64 at = ((i64)grp * 32 + 8 * j + (lane >> 2)) * 4 + g2;
          sc[j] = spilled ? my_spill[at] : scores[at];
        }
        __syncwarp();
        uint8_t* pt = reinterpret_cast<uint8_t*>(scores) + (size_t)place * 1024;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kl = 8 * j + (lane >> 2);
          const i64 key = (i64)grp * 32 + kl;
          i64 pv = 0;
          if (key < hi && key <= qp2) pv = attn_weight_any(p, sc[j], mx, rowshift);
          den += pv;
          int pr = (int)pv;
          const int off = (kl >> 4) * 256 + (kl & 15) + g2 * 16;
          pt[off] = (uint8_t)split8(pr);                              // row g      (limb 0)
          pt[off + 64] = (uint8_t)split8(pr);                         // row 4 + g  (limb 1)
          pt[off + 128] = (uint8_t)split8(pr);                        // row 8 + g  (limb 2)
        }
        fence_proxy_async_smem();                                     // the tile is read by tcgen05 (async proxy)
        __syncwarp();
        if (lane == 0) flag_release(&sm->ptag[place], wave + ck + 1);
      }
    }
    gidx += (uint32_t)nst;                                            // the V stages belong to the MMA warp

    den += __shfl_xor_sync(0xffffffffu, den, 4);
    den += __shfl_xor_sync(0xffffffffu, den, 8);
    den += __shfl_xor_sync(0xffffffffu, den, 16);
    if (lane < 4) sm->pden[warp][lane] = den;

    // ---- accumulators: first tile lanes 0..63 = (V limb 0, dim), 64..127 = (V limb 1, dim); second tile lanes
    //      64..127 = (V limb 2, dim). Column 4 i + g = (p limb i, query g). ----
    i64 part[4] = {0, 0, 0, 0};
    if (warp < 4) {
      bool done = ok && nst > 0;
      if (done) done = mbar_wait(&sm->acc_done, (wave + nchunks - 1) & 1);
      done = done && (*abort_flag == 0);
      done = __all_sync(0xffffffffu, done);
      if (done) {
        tc_fence_after();
        uint32_t d01[16], d12[16];
        const uint32_t tb = tmem + ((uint32_t)(warp * 32) << 16);
        tmem_ld16(tb, d01);
        tmem_ld16(tb + 16, d12);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          i64 a = (i64)(int32_t)d01[g] + shl((i64)(int32_t)d01[4 + g], 8) + shl((i64)(int32_t)d01[8 + g], 16);
          if (warp >= 2) {
            const i64 b = (i64)(int32_t)d12[g] + shl((i64)(int32_t)d12[4 + g], 8) + shl((i64)(int32_t)d12[8 + g], 16);
            a = shl(a, 8) + shl(b, 16);
          }
          part[g] = a;
        }
      } else if (nst > 0) {
        ok = false;
      }
      tc_fence_before();
    }
    if (warp < 2) {
#pragma unroll
      for (int g = 0; g < 4; ++g) sm->cnum[g][warp * 32 + lane] = part[g];
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");     // cnum, pden written; accumulators and p tiles read
    if (warp >= 2 && warp < 4) {
      const int d = (warp - 2) * 32 + lane;
#pragma unroll
      for (int g = 0; g < 4; ++g)
        if (g < p.M) p.num[(pz * p.M + g) * ATT_HD + d] = sm->cnum[g][d] + part[g];
    }
    if (threadIdx.x < p.M) {
      i64 t = 0;
      for (int w = 0; w < NW; ++w) t += sm->pden[w][threadIdx.x];
      p.den[pz * p.M + threadIdx.x] = t;
    }
    wave += (uint32_t)nchunks;
    asm volatile("bar.sync 1, %0;" ::"r"(CTHREADS) : "memory");     // cnum / pden / wmax are free for the next pair
  }
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, ATT3_TMEM_COLS);
  }
}

}  // namespace bx
