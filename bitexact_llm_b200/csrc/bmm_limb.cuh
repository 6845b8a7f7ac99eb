// The exact batched integer product `bmm` (src/bitexact/bmm.py:78-102) on the tcgen05 limb main loop: up to 3 x 3
// int8 limb products into five int32 TMEM accumulators (one per limb weight), joined to int64 once at the end, as the
// reference's Triton kernel does with tl.dot (src/bitexact/bmm.py:27-75).
//
// Two steps. bmm_pack_kernel turns an operand with arbitrary element strides into K-major limb planes
// int8 [3, Z R, K16] (R rows per batch, K padded with zeros to a multiple of 16: the TMA row pitch), reading b
// transposed where needed. bmm_limb_kernel<TA> then runs limb_gemm_tile with the planes of b^T as its 128-row
// operand and TA rows of a as its stacked operand; one CTA per (batch, 128 columns of b, TA rows of a). A tile that
// reaches past its batch reads rows of the next one (or zeros past the end): those outputs are not stored.
#pragma once

#include "bx_rules.cuh"
#include "limb_gemm.cuh"

namespace bx {

struct BmmEpiParams {
  int64_t* c;            // [Z, M, N]
  int M, N;              // per batch
};

template <int TA>
struct BmmEpilogue {
  using Params = BmmEpiParams;
  static constexpr int CW = (TA % (8 * EPI_GROUPS) == 0) ? 8 : 4;
  struct Row {
    int z, n, m_first;   // batch, column of b (local), first row of a of this tile (local)
    bool nok;
  };

  // n0g / m0g: row origins in the stacked planes (z N + local, z M + local); a tile starts inside its batch.
  static __device__ __forceinline__ Row load_row(int quarter, int, int lane, int n0g, int m0g, const Params& p) {
    Row r;
    r.z = n0g / p.N;
    r.n = n0g - r.z * p.N + quarter * 32 + lane;
    r.m_first = m0g - r.z * p.M;
    r.nok = r.n < p.N;
    return r;
  }
  static __device__ __forceinline__ void prefetch(const Row&, int, int, int, const Params&) {}

  static __device__ __forceinline__ void run(uint32_t tmem, int quarter, int group, int, int, int, bool has_k,
                                             const Params& p, const Row& r) {
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
    i64* cz = reinterpret_cast<i64*>(p.c) + (i64)r.z * p.M * p.N;
#pragma unroll 1
    for (int c0 = group * CW; c0 < TA; c0 += CW * EPI_GROUPS) {
      if (r.m_first + c0 >= p.M) break;              // warp-uniform
      uint32_t acc[5][CW];
#pragma unroll
      for (int b = 0; b < 5; ++b) tmem_ldn<CW>(tbase + b * TA + c0, acc[b]);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < CW; ++i) {
        const int m = r.m_first + c0 + i;
        if (m < p.M && r.nok)
          cz[(i64)m * p.N + r.n] = has_k ? join5(acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i]) : 0;
      }
    }
  }
};

// grid.x = (batch, tile of b columns, tile of a rows), the a-row tile fastest.
template <int TA>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
bmm_limb_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_a,
                const BmmEpiParams ep, int K16, int n_tiles, int m_tiles) {
  const int mt = blockIdx.x % m_tiles;
  const int nt = (blockIdx.x / m_tiles) % n_tiles;
  const int z = blockIdx.x / (m_tiles * n_tiles);
  limb_gemm_tile<3, 3, TA, BmmEpilogue<TA>>(&tmap_b, &tmap_a, z * ep.N + nt * WROWS, z * ep.M + mt * TA, 0,
                                            (K16 + BKB - 1) / BKB, ep);
}

// x[z, r, k] at x + z sz + r sr + k sk (elements) -> planes int8 [3, Z R, K16], zeros for k >= K. One thread per 16
// consecutive k of one row: a 16-byte store per plane.
template <class TX>
__global__ void bmm_pack_kernel(const TX* __restrict__ x, int64_t sz, int64_t sr, int64_t sk, int8_t* __restrict__ planes,
                                int Z, int R, int K, int K16) {
  const int64_t per_row = K16 / 16;
  const int64_t rows = (int64_t)Z * R;
  const int64_t total = rows * per_row;
  const int64_t plane = rows * K16;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = t / per_row;
    const int k0 = (int)(t % per_row) * 16;
    const int64_t z = row / R, r = row % R;
    const TX* src = x + z * sz + r * sr;
    uint32_t out[3][4];
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = k0 + 4 * v + i;
        int e = k < K ? (int)src[(int64_t)k * sk] : 0;
        w0 |= (uint32_t)(split8(e) & 255) << (8 * i);
        w1 |= (uint32_t)(split8(e) & 255) << (8 * i);
        w2 |= (uint32_t)(split8(e) & 255) << (8 * i);
      }
      out[0][v] = w0; out[1][v] = w1; out[2][v] = w2;
    }
#pragma unroll
    for (int l = 0; l < 3; ++l)
      *reinterpret_cast<uint4*>(planes + l * plane + row * K16 + k0) = make_uint4(out[l][0], out[l][1], out[l][2], out[l][3]);
  }
}

}  // namespace bx
