// Exact-mode linear y = round((q @ W_bf16^T) * 2^(sh + 24)) as one kernel: 3x3 int8 limb products on tcgen05 into
// five int32 TMEM accumulators, int64 join, sparse low-bit residual, one round-half-up, lost-bit flag.
//
// Replaces, with the same integers: FusedLin.__call__ / _lin_kernel (src/bitexact/vllm_plugin/exact_gemm.py:58-119,
// 284-316) = wmm (src/bitexact/exact/wmm.py:31-121) + residual (:124-129) + epilogue (:132-150).
#pragma once

#include "bx_rules.cuh"
#include "limb_gemm.cuh"
#include "limb_gemm_pair.cuh"


namespace bx {

struct ExactEpiParams {
  const int32_t* q;      // [M, ldq] activations (residual gather)
  int64_t ldq;
  const int64_t* sh;     // [M] row exponents
  const int64_t* d;      // [N] residual grid offset, 0..30
  const int64_t* g;      // [N] row grid exponent
  const int32_t* cnt;    // [N] residual entries per weight row (may be null: no residual)
  const int32_t* ec;     // [N, R] residual columns
  const int64_t* ev;     // [N, R] residual values
  int R;
  int64_t* y;            // [M, N]
  int32_t* flag;         // sticky lost-bit / range flag (only ever set to 1)
  int M, N;
  int checked;
};

template <int TA>
struct ExactEpilogue {
  using Params = ExactEpiParams;

  static constexpr int RMAX = 2;

  // What a thread needs about its weight row n (TMEM lane): loaded BEFORE the accumulators are waited for, so the
  // loads (two dependent levels: the count, then the list) overlap the main loop instead of heading every tile's
  // epilogue. The residual list of row n (a handful of entries in a few per cent of the rows) is read once.
  static constexpr int NS = (TA + 31) / 32;
  struct Row {
    int n, d, cnt, wcnt;
    bool nok;
    i64 gd;
    int ecr[RMAX];
    i64 evr[RMAX];
    i64 shv[NS];             // row exponents of the tile's activation rows, lane-held (lane_slot)
  };

  static __device__ __forceinline__ Row load_row(int quarter, int group, int lane, int n0, int m0, const Params& p) {
    Row r;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int c = s * 32 + lane;
      r.shv[s] = (c < TA && m0 + c < p.M) ? p.sh[m0 + c] : 0;
    }
    r.n = n0 + quarter * 32 + lane;
    r.nok = r.n < p.N;
    r.d = r.nok ? (int)p.d[r.n] : 0;
    r.gd = r.nok ? p.g[r.n] - (i64)r.d + FR : 0;
    r.cnt = (r.nok && p.cnt) ? p.cnt[r.n] : 0;
#pragma unroll
    for (int j = 0; j < RMAX; ++j) {
      r.ecr[j] = 0;
      r.evr[j] = 0;
      if (j < r.cnt) {
        r.ecr[j] = p.ec[(i64)r.n * p.R + j];
        r.evr[j] = p.ev[(i64)r.n * p.R + j];
      }
    }
    r.wcnt = __reduce_max_sync(0xffffffffu, r.cnt);                    // longest list in the warp (uniform)
    return r;
  }

  // Pulls the gathers from q of a thread whose weight row has a residual list into L1 while the tile's MMAs still
  // run.
  static __device__ __forceinline__ void prefetch(const Row& r, int group, int lane, int m0, const Params& p) {
#pragma unroll 1
    for (int c0 = group * CW; c0 < TA; c0 += CW * EPI_GROUPS) {
      if (m0 + c0 >= p.M) break;
      if (r.cnt > 0) {
        for (int i = 0; i < CW; ++i) {
          const int m = m0 + c0 + i;
          if (m >= p.M) break;
#pragma unroll
          for (int j = 0; j < RMAX; ++j)
            if (j < r.cnt) prefetch_l1(p.q + (i64)m * p.ldq + r.ecr[j]);
        }
      }
    }
  }

  // Accumulator columns per chunk: 8 when the TA columns split evenly over the EPI_GROUPS warps of a lane quarter in
  // chunks of 8, else 4 (TA = 48: three chunks of 4 for every warp instead of two chunks of 8 for half of them).
  static constexpr int CW = (TA % (8 * EPI_GROUPS) == 0) ? 8 : 4;

  static constexpr int NCH = (TA + CW * EPI_GROUPS - 1) / (CW * EPI_GROUPS);      // chunks per warp

  // One thread per weight row n (TMEM lane) and column group; walks its share of the TA activation rows in chunks
  // of CW accumulator columns. A thread whose weight row has a residual list does not finish its outputs here: each
  // would wait for its own gather from q, one after the other, with the rest of the warp waiting beside it. It
  // stores the joined sum T in place of y, and the warp then deals these (row, column) outputs out over its 32
  // lanes (`deferred`): all their loads are in flight together, one round trip instead of one per column.
  static __device__ __forceinline__ void run(uint32_t tmem, int quarter, int group, int lane, int n0, int m0,
                                             bool has_k, const Params& p, const Row& r) {
    const int n = r.n;
    const bool listed = r.cnt > 0 && r.nok;
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
    bool any_bad = false;
#pragma unroll 1
    for (int c0 = group * CW; c0 < TA; c0 += CW * EPI_GROUPS) {
      if (m0 + c0 >= p.M) break;                     // warp-uniform
      const i64 sh_slot = lane_slot<NS>(r.shv, c0);      // lane (c0 & 31) + i holds the exponent of row c0 + i
      uint32_t acc[5][CW];
#pragma unroll
      for (int b = 0; b < 5; ++b) tmem_ldn<CW>(tbase + b * TA + c0, acc[b]);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < CW; ++i) {
        const int m = m0 + c0 + i;
        const bool in = m < p.M && r.nok;
        const i64 pv = __shfl_sync(0xffffffffu, sh_slot, (c0 & 31) + i) + r.gd;
        const i64 T = has_k ? join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]) : 0;
        bool bad;
        const i64 yv = round_rule_warp(T, 0, r.d, pv, in && !listed, bad);
        any_bad |= bad;
        if (in) p.y[(i64)m * p.N + n] = listed ? T : yv;
      }
    }
    if (r.wcnt > 0) deferred(group, lane, m0, p, r, any_bad);         // warp-uniform
    if (p.checked && any_bad) *p.flag = 1;
  }

  // The outputs of the warp's weight rows with a residual list: item (l, cc) = l-th such row, cc-th column of the
  // warp, one item per lane and round. The owner's constants come by shuffle, T is read back from y.
  static __device__ __forceinline__ void deferred(int group, int lane, int m0, const Params& p, const Row& r,
                                                  bool& any_bad) {
    constexpr unsigned FULL = 0xffffffffu;
    const unsigned lmask = __ballot_sync(FULL, r.cnt > 0 && r.nok);
    if (lmask == 0) return;
    __threadfence_block();                            // the sums stored above are read by other lanes below
    __syncwarp();
    constexpr int NCOL = NCH * CW;
    const int items = __popc(lmask) * NCOL;
    for (int it0 = 0; it0 < items; it0 += 32) {
      const int it = it0 + lane;
      const bool has = it < items;
      const int l = has ? it / NCOL : 0, cc = has ? it % NCOL : 0;
      const int src = __fns(lmask, 0, l + 1);        // lane of the l-th listed row
      const int c = ((cc / CW) * EPI_GROUPS + group) * CW + cc % CW;
      const int m = m0 + c;
      const bool on = has && c < TA && m < p.M;
      const int n = __shfl_sync(FULL, r.n, src), d = __shfl_sync(FULL, r.d, src), cnt = __shfl_sync(FULL, r.cnt, src);
      const i64 gd = __shfl_sync(FULL, r.gd, src);
      i64 shm = 0;
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const i64 v = __shfl_sync(FULL, r.shv[s], c & 31);
        if ((c >> 5) == s) shm = v;
      }
      int ec0[RMAX];
      i64 ev0[RMAX];
#pragma unroll
      for (int j = 0; j < RMAX; ++j) {
        ec0[j] = __shfl_sync(FULL, r.ecr[j], src);
        ev0[j] = __shfl_sync(FULL, r.evr[j], src);
      }
      i64 T = 0, B = 0;
      if (on) {
        T = p.y[(i64)m * p.N + n];
#pragma unroll
        for (int j = 0; j < RMAX; ++j)
          if (j < cnt) B += (i64)p.q[(i64)m * p.ldq + ec0[j]] * ev0[j];
        for (int j = RMAX; j < cnt; ++j)
          B += (i64)p.q[(i64)m * p.ldq + p.ec[(i64)n * p.R + j]] * p.ev[(i64)n * p.R + j];
      }
      bool bad;
      const i64 yv = round_rule_warp(T, B, d, shm + gd, on, bad);
      any_bad |= bad;
      if (on) p.y[(i64)m * p.N + n] = yv;
    }
  }
};

template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
exact_linear_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                    const ExactEpiParams ep, int K, int m_tiles) {
  const int mt = blockIdx.x % m_tiles;
  const int nt = blockIdx.x / m_tiles;
  limb_gemm_tile<3, 3, TA, ExactEpilogue<TA>>(&tmap_w, &tmap_a, nt * WROWS, mt * TA, 0, (K + BKB - 1) / BKB, ep);
}

// Persistent form (one CTA per SM, double-buffered accumulators): used when the tile list is longer than one wave.
template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
exact_linear_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                               const ExactEpiParams ep, int K, int n_tiles, int m_tiles) {
  limb_gemm_persistent<3, 3, TA, ExactEpilogue<TA>>(&tmap_w, &tmap_a, n_tiles, m_tiles, (K + BKB - 1) / BKB, ep);
}

// CTA-pair form (tcgen05 .cta_group::2, see limb_gemm_pair.cuh): a cluster of two CTAs per 256 weight rows, one pair
// per TPC walks the tile list. tmap_b is the activation map with boxes of TA / 2 rows of one limb plane.
template <int TA>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
exact_linear_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_b,
                         const ExactEpiParams ep, int K, int n_tiles2, int m_tiles) {
  limb_gemm_pair_persistent<3, 3, TA, ExactEpilogue<TA>>(&tmap_w, &tmap_b, n_tiles2, m_tiles, (K + BKB - 1) / BKB, ep);
}

// q int32 [M, K] (row stride ldq) -> limb planes int8 [3, M, K] (signed base-256 digits, intops.py:62-70).
__global__ void split_limbs_kernel(const int32_t* __restrict__ q, int64_t ldq, int8_t* __restrict__ a8, int M, int K) {
  const int64_t per_row = K / 16;
  const int64_t total = (int64_t)M * per_row;
  const int64_t plane = (int64_t)M * K;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = t / per_row, c = (t % per_row) * 16;
    const int4* src = reinterpret_cast<const int4*>(q + m * ldq + c);
    uint32_t out[3][4];
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int4 x = src[v];
      int e[4] = {x.x, x.y, x.z, x.w};
      uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int r = e[i];
        w0 |= (uint32_t)(split8(r) & 255) << (8 * i);
        w1 |= (uint32_t)(split8(r) & 255) << (8 * i);
        w2 |= (uint32_t)(split8(r) & 255) << (8 * i);
      }
      out[0][v] = w0; out[1][v] = w1; out[2][v] = w2;
    }
#pragma unroll
    for (int l = 0; l < 3; ++l)
      *reinterpret_cast<uint4*>(a8 + l * plane + m * K + c) = make_uint4(out[l][0], out[l][1], out[l][2], out[l][3]);
  }
}

}  // namespace bx
