// Split-K form of the int8-mode fused linear (GEMM + post): the cluster kernel of exact_linear_splitk.cuh with the
// int8 policy. One weight limb against two activation limbs, two TMEM column blocks; a K slice's partial is
// c0 + (c1 << 8) as int64 (sums of slices are sums of these, exact in any order), the owner of a column applies
// segs.post (src/bitexact/int8/segs.py:62-67) to the total. For projections with few weight tiles and long K: the
// down projection (N = 2048, K = 8192) has 16 weight tiles, and with its output columns sharded over GPUs
// (N = 512 per rank at 4 GPUs) only 4.
#pragma once

#include "exact_linear_splitk.cuh"
#include "int8_linear.cuh"

namespace bx {

template <int TA>
struct Int8SplitEpi {
  using Params = Int8EpiParams;
  static constexpr int NW = 1, NA = 2, NS = (TA + 31) / 32;
  struct Consts {
    int n;
    bool nok;
    i64 mc;
    i64 mant[NS], e[NS];                                              // the tile's row scales, lane-held
  };

  static __device__ __forceinline__ Consts load(int n0, int m0, int quarter, int, int lane, int, int, const Params& ep) {
    Consts c;
    c.n = n0 + quarter * 32 + lane;
    c.nok = c.n < ep.N;
    c.mc = c.nok ? ep.mul[c.n] : 0;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int col = s * 32 + lane;
      const bool on = col < TA && m0 + col < ep.M;
      c.mant[s] = on ? ep.mant[m0 + col] : 0;
      c.e[s] = on ? ep.e[m0 + col] : 0;
    }
    return c;
  }

  static __device__ __forceinline__ i64 join(const uint32_t (&acc)[2][8], int i) {
    return (i64)(int32_t)acc[0][i] + shl((i64)(int32_t)acc[1][i], 8);
  }

  static __device__ __forceinline__ int a_rows(const Params& ep) { return ep.M; }

  static __device__ __forceinline__ void final(i64 T, int col, int m, const Consts& c, const Params& ep, bool& any_bad) {
    const i64 mant_m = __shfl_sync(0xffffffffu, lane_slot<NS>(c.mant, col), col & 31);
    const i64 e_m = __shfl_sync(0xffffffffu, lane_slot<NS>(c.e, col), col & 31);
    if (c.nok) {
      bool bad;
      ep.y[(i64)m * ep.N + c.n] = int8_post(T, c.mc, ep.fmsh, mant_m, e_m, bad);
      any_bad |= bad;
    }
  }

  static __device__ __forceinline__ void finish(bool any_bad, const Params& ep) {
    if (ep.checked && any_bad) *ep.flag = 1;
  }
};

template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
int8_linear_splitk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                          const Int8EpiParams ep, int K, int m_tiles) {
  limb_splitk<TA, Int8SplitEpi<TA>>(tmap_w, tmap_a, ep, K, m_tiles);
}

}  // namespace bx
