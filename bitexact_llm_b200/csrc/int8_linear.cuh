// int8-mode linear on the same tcgen05 main loop: ONE weight limb (int8 weights, per-channel multiplier) against
// TWO activation limbs (|q| <= 127 * 256). One MMA per 32-deep K slice with N = 2 TA: TMEM column block 0 holds
// the limb-0 products, block 1 the limb-1 products; acc = c0 + (c1 << 8).
//
// Two epilogues:
//   Int8RawEpilogue   stores the int32 limb products like torch._int_mm on stacked limbs
//                     (int_mm, src/bitexact/int8/gemm_skinny.py:80-97): c[i * M + m, n] = block i.
//   Int8PostEpilogue  fuses segs.post (src/bitexact/int8/segs.py:62-67; fused copy _y,
//                     src/bitexact/vllm_plugin/tri_fuse.py:74-79): t = rsh(acc * m_c, fmsh),
//                     y = rsh(t * mant_r, 8 - e_r); flag when |t| >= 2^38.
#pragma once

#include "bx_rules.cuh"
#include "limb_gemm.cuh"

namespace bx {

// torch's shift rules for int64 tensors, as the reference's kernels restate them
// (src/bitexact/vllm_plugin/tri_mlp.py:36-54): x >> s saturates at 63, x << s gives 0 from 64 on.
__device__ __forceinline__ i64 shr_t(i64 x, i64 s) { return x >> (int)imin(s, 63); }
__device__ __forceinline__ i64 shl_t(i64 x, i64 s) { return s >= 64 ? 0 : shl(x, (int)s); }
// intops.rsh with a tensor shift (src/bitexact/intops.py:24-34): round half up for s > 0, multiply for s <= 0.
__device__ __forceinline__ i64 rsh_t(i64 x, i64 s) {
  const i64 pos = imax(s, 0), neg = imax(-s, 0);
  const i64 half = pos > 0 ? shl_t(1, pos - 1) : 0;
  return shl_t(shr_t(x + half, pos), neg);
}

// rsh_t for a shift known to lie in 1 .. 62: the same integers without the generality.
__device__ __forceinline__ i64 rsh_pos(i64 x, int s) { return (x + (1ll << (s - 1))) >> s; }

// segs.post on a joined accumulator: t = rsh(acc * m_c, fmsh), y = rsh(t * mant_r, 8 - e_r); bad when |t| >= 2^38.
// Both shifts are almost always in 1 .. 62 (fmsh is a constant of the layer, 8 - e_r a property of the activation
// row, the same for every lane of a warp): that case takes two plain rounding shifts, any other the general rule.
__device__ __forceinline__ i64 int8_post(i64 acc, i64 mc, i64 fmsh, i64 mant, i64 e, bool& bad) {
  const i64 s2 = 8 - e;
  if (fmsh >= 1 && fmsh <= 62 && s2 >= 1 && s2 <= 62) {               // warp-uniform
    const i64 t = rsh_pos((i64)((u64)acc * (u64)mc), (int)fmsh);
    bad = iabs(t) >= (1ll << 38);
    return rsh_pos((i64)((u64)t * (u64)mant), (int)s2);
  }
  const i64 t = rsh_t((i64)((u64)acc * (u64)mc), fmsh);
  bad = iabs(t) >= (1ll << 38);
  return rsh_t((i64)((u64)t * (u64)mant), s2);
}

struct Int8EpiParams {
  int32_t* c;            // raw: [R, N] int32, limb i of row m at row i * M + m
  const int64_t* mul;    // post: [N] per-channel multipliers
  int64_t fmsh;          // post: scalar shift
  const int64_t* mant;   // post: [M] row scale mantissa in [2^23, 2^24]
  const int64_t* e;      // post: [M] row scale exponent
  int64_t* y;            // post: [M, N] at 16 fractional bits
  int32_t* flag;         // post: sticky |t| >= 2^38 flag
  int M, N;
  int checked;
};

template <int TA, bool POST>
struct Int8Epilogue {
  using Params = Int8EpiParams;

  // The thread's weight row and its channel multiplier, loaded before the accumulators are waited for.
  static constexpr int NS = (TA + 31) / 32;
  struct Row {
    int n;
    bool nok;
    i64 mc;
    i64 mant[NS], e[NS];     // row scales of the tile's activation rows, lane-held (lane_slot)
  };

  static __device__ __forceinline__ Row load_row(int quarter, int group, int lane, int n0, int m0, const Params& p) {
    Row r;
    r.n = n0 + quarter * 32 + lane;
    r.nok = r.n < p.N;
    r.mc = (POST && r.nok) ? p.mul[r.n] : 0;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int c = s * 32 + lane;
      const bool on = POST && c < TA && m0 + c < p.M;
      r.mant[s] = on ? p.mant[m0 + c] : 0;
      r.e[s] = on ? p.e[m0 + c] : 0;
    }
    return r;
  }

  static __device__ __forceinline__ void prefetch(const Row&, int, int, int, const Params&) {}

  static __device__ __forceinline__ void run(uint32_t tmem, int quarter, int group, int lane, int n0, int m0,
                                             bool has_k, const Params& p, const Row& r) {
    const int n = r.n;
    const bool nok = r.nok;
    const i64 mc = r.mc;
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
    bool any_bad = false;
#pragma unroll 1
    for (int c0 = group * 8; c0 < TA; c0 += 8 * EPI_GROUPS) {
      if (m0 + c0 >= p.M) break;
      uint32_t a0[8], a1[8];
      tmem_ld8(tbase + c0, a0);
      tmem_ld8(tbase + TA + c0, a1);
      const i64 mant_slot = POST ? lane_slot<NS>(r.mant, c0) : 0, e_slot = POST ? lane_slot<NS>(r.e, c0) : 0;
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = m0 + c0 + i;
        const i64 mant_m = POST ? __shfl_sync(0xffffffffu, mant_slot, (c0 & 31) + i) : 0;
        const i64 e_m = POST ? __shfl_sync(0xffffffffu, e_slot, (c0 & 31) + i) : 0;
        if (m < p.M && nok) {
          const int32_t v0 = has_k ? (int32_t)a0[i] : 0, v1 = has_k ? (int32_t)a1[i] : 0;
          if (POST) {
            bool bad;
            p.y[(i64)m * p.N + n] = int8_post((i64)v0 + shl((i64)v1, 8), mc, p.fmsh, mant_m, e_m, bad);
            any_bad |= bad;
          } else {
            p.c[(i64)m * p.N + n] = v0;
            p.c[((i64)p.M + m) * p.N + n] = v1;
          }
        }
      }
    }
    if (POST && p.checked && any_bad) *p.flag = 1;
  }
};

template <int TA, bool POST>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
int8_linear_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                   const Int8EpiParams ep, int K, int m_tiles) {
  const int mt = blockIdx.x % m_tiles;
  const int nt = blockIdx.x / m_tiles;
  limb_gemm_tile<1, 2, TA, Int8Epilogue<TA, POST>>(&tmap_w, &tmap_a, nt * WROWS, mt * TA, 0, (K + BKB - 1) / BKB, ep);
}

// Persistent form (one CTA per SM walks the tile list, two accumulator buffers: the post epilogue of tile i overlaps
// the MMAs of tile i + 1). 2 * 2 TA <= 512 TMEM columns holds for every TA up to 128.
template <int TA, bool POST>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
int8_linear_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                              const Int8EpiParams ep, int K, int n_tiles, int m_tiles) {
  limb_gemm_persistent<1, 2, TA, Int8Epilogue<TA, POST>>(&tmap_w, &tmap_a, n_tiles, m_tiles, (K + BKB - 1) / BKB, ep);
}

}  // namespace bx
