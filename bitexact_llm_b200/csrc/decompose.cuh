// Weight preparation of exact mode on the device: bf16 [N, K] -> 3 dense int8 limb planes + per-row grid exponents
// + the sparse low-bit residual, one CTA per weight row.
//
// Per output row (src/bitexact/exact/consts.py:67-107 of the reference): the grid exponent g is the smallest
// exponent for which every |trunc(w / 2^g)| <= 8355711 (three signed base-256 digits); the bits that a truncation
// drops are kept exactly as integers on the finer grid g - d, d chosen so that the lowest dropped bit of the row is
// representable. Row-parallel integer work: nothing crosses rows, so the tensors are those of the host code whatever
// the grid. Load-time step, bound by the 2 bytes read + 3 bytes written per weight.
//
// decompose_rows_kernel: limbs, g, d and the number of residual entries of each row.
// decompose_residual_kernel: the entries (row, column, value) in row-major order at the row's offset (the caller's
// exclusive prefix sum of the counts), i.e. the coordinate list the host code produces.
#pragma once

#include "bx_rules.cuh"

namespace bx {

constexpr int DEC_THREADS = 256;
constexpr int DEC_LIM3 = 8355711;
constexpr int DEC_FLAG_NONFINITE = 1, DEC_FLAG_FINE = 2, DEC_FLAG_LIMBS = 4;

// bf16 bits -> magnitude of the significand (0..255) and exponent, w = +-mag * 2^ex exactly (consts.py:33-42).
__device__ __forceinline__ void bf16_parts(uint32_t b, int& mag, int& ex, bool& neg, bool& nonfinite) {
  const int e = (b >> 7) & 0xFF;
  const int frac = b & 0x7F;
  nonfinite = e == 255;
  mag = e > 0 ? (frac | 0x80) : frac;
  ex = (e > 0 ? e : 1) - 134;
  neg = (b & 0x8000u) != 0;
}

// Largest s >= 0 with mag << s <= 8355711 (mag in 1..255).
__device__ __forceinline__ int dec_smax(int mag) {
  int s = 22 - (31 - __clz(mag));                       // top bit at position 22
  if ((mag << s) > DEC_LIM3) --s;
  return s;
}

__device__ __forceinline__ int block_reduce_int(int v, int* red, bool is_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? max(v, u) : min(v, u);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[0];
#pragma unroll
  for (int w = 1; w < DEC_THREADS / 32; ++w) v = is_max ? max(v, red[w]) : min(v, red[w]);
  return v;
}

// The dense truncation and what it drops, on the grid 2^g.
__device__ __forceinline__ void dec_dense(int mag, int ex, int g, int& dense, int& lost) {
  const int sh = ex - g;
  if (sh >= 0) {
    dense = mag << min(sh, 22);                         // g >= ex - smax(mag): at most 22 places
    lost = 0;
  } else {
    const int r = min(-sh, 31);
    dense = mag >> r;
    lost = mag - (dense << r);
  }
}

// grid N: limbs [3][N][K] (plane stride N K), g, d, cnt of row blockIdx.x; flag |= DEC_FLAG_* on bad input.
__global__ void __launch_bounds__(DEC_THREADS) decompose_rows_kernel(const uint16_t* __restrict__ w, i64 ldw,
                                                                      int8_t* __restrict__ limbs, i64* __restrict__ g_out,
                                                                      i64* __restrict__ d_out, int32_t* __restrict__ cnt_out,
                                                                      int32_t* flag, int N, int K) {
  __shared__ int red[DEC_THREADS / 32];
  const i64 row = blockIdx.x;
  const uint16_t* wr = w + row * ldw;
  constexpr int NONE = -1000000;
  int need = NONE;
  bool bad = false;
  for (int c = threadIdx.x; c < K; c += DEC_THREADS) {
    int mag, ex;
    bool neg, nf;
    bf16_parts(wr[c], mag, ex, neg, nf);
    bad |= nf;
    if (mag > 0) need = max(need, ex - dec_smax(mag));
  }
  int g = block_reduce_int(need, red, true);
  if (g == NONE) g = 0;
  int low = 1000000, cnt = 0;
  bool rem_bad = false;
  const i64 plane = (i64)N * K;
  int8_t* lr = limbs + row * K;
  for (int c = threadIdx.x; c < K; c += DEC_THREADS) {
    int mag, ex, dense, lost;
    bool neg, nf;
    bf16_parts(wr[c], mag, ex, neg, nf);
    dec_dense(mag, ex, g, dense, lost);
    if (lost > 0) {
      low = min(low, ex + (__ffs(lost) - 1));
      ++cnt;
    }
    int rem = neg ? -dense : dense;
    lr[c] = (int8_t)split8(rem);
    lr[plane + c] = (int8_t)split8(rem);
    lr[2 * plane + c] = (int8_t)split8(rem);
    rem_bad |= rem != 0;
  }
  low = block_reduce_int(low, red, false);
  const int gf = min(low, g);
  // the count: a block sum through the same shared words
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
#pragma unroll
    for (int k = 0; k < DEC_THREADS / 32; ++k) total += red[k];
    g_out[row] = g;
    d_out[row] = g - gf;
    cnt_out[row] = total;
    if (g - gf > 30) atomicOr(flag, DEC_FLAG_FINE);
  }
  if (bad) atomicOr(flag, DEC_FLAG_NONFINITE);
  if (rem_bad) atomicOr(flag, DEC_FLAG_LIMBS);
}

// grid N: the residual entries of row blockIdx.x, in column order, at start[row]: rr = row, rc = column,
// rv = +-(dropped bits) on the grid g - d (consts.py:97-104).
__global__ void __launch_bounds__(DEC_THREADS) decompose_residual_kernel(const uint16_t* __restrict__ w, i64 ldw,
                                                                          const i64* __restrict__ g_in,
                                                                          const i64* __restrict__ d_in,
                                                                          const i64* __restrict__ start,
                                                                          i64* __restrict__ rr, i64* __restrict__ rc,
                                                                          i64* __restrict__ rv, int K) {
  __shared__ int wsum[DEC_THREADS / 32];
  __shared__ int base_s;
  const i64 row = blockIdx.x;
  const uint16_t* wr = w + row * ldw;
  const int g = (int)g_in[row], gf = g - (int)d_in[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < K; c0 += DEC_THREADS) {
    const int c = c0 + threadIdx.x;
    int mag = 0, ex = 0, dense, lost = 0;
    bool neg = false, nf;
    if (c < K) {
      bf16_parts(wr[c], mag, ex, neg, nf);
      dec_dense(mag, ex, g, dense, lost);
    }
    const unsigned m = __ballot_sync(0xffffffffu, lost > 0);
    if (lane == 0) wsum[warp] = __popc(m);
    __syncthreads();
    int off = base_s;
    for (int k = 0; k < warp; ++k) off += wsum[k];
    if (lost > 0) {
      const i64 at = start[row] + off + __popc(m & ((1u << lane) - 1));
      const int s = ex - gf;
      const i64 v = s >= 0 ? ((i64)lost << s) : ((i64)lost >> (-s));
      rr[at] = row;
      rc[at] = c;
      rv[at] = neg ? -v : v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
#pragma unroll
      for (int k = 0; k < DEC_THREADS / 32; ++k) t += wsum[k];
      base_s += t;
    }
    __syncthreads();
  }
}

}  // namespace bx
