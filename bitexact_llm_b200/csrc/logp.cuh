// Integer log p of given tokens from int64 logits rows [M, V] at fr fractional bits.
//
// log p(tok) = (l_tok - max) - ln(sum_v e^(l_v - max)), everything an int64: the terms e^z come from a table of e^x
// at 44 bits with step 2^-12 over [-40, 0] (linear interpolation on the fr - 12 low bits, rounded; arguments below
// -40 take the first entry), their sum S is < 2^62 and exact in any order, ln S comes from the sampler's ln table.
// The result is an integer at 2^-40. Same integers as int_logp (src/bitexact/vllm_plugin/rl.py:43-65) and as the
// chunked two-pass form of src/bitexact/vllm_plugin/tri_logp.py:27-91.
//
// Two passes over the rows (bound by HBM: 2 x 8 M V bytes): logp_max_kernel reduces every (row, column chunk) to
// its maximum, logp_sum_kernel first folds the row's chunk maxima (or takes a row maximum given by the caller: a
// column shard sums against the maximum of the full row), then sums its chunk's terms. logp_finish_kernel works on
// [M]: the sum over the chunks, ln S and the target term.
#pragma once

#include "sampler.cuh"

namespace bx {

constexpr int LOGP_THREADS = 256;
constexpr int LSE_FE = 44, LSE_MIN = -40, LSE_STEP = 12;
constexpr int LSE_LAST = -LSE_MIN << LSE_STEP;             // index of e^0 = the last table entry
constexpr i64 LOGP_INVALID = (i64)(-0x7fffffffffffffffll - 1);

__device__ __forceinline__ i64 block_max_i64(i64 v, i64* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = imax(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = red[0];
#pragma unroll
  for (int w = 1; w < LOGP_THREADS / 32; ++w) v = imax(v, red[w]);
  return v;
}

// grid (nch, M): pmax[row * nch + chunk] = max of logits[row, chunk columns].
__global__ void __launch_bounds__(LOGP_THREADS) logp_max_kernel(const i64* __restrict__ lg, i64 ld, i64* __restrict__ pmax,
                                                                 int V, int ch, int nch) {
  __shared__ i64 red[LOGP_THREADS / 32];
  const int row = blockIdx.y, c0 = blockIdx.x * ch, c1 = min(c0 + ch, V);
  const i64* x = lg + (i64)row * ld;
  i64 v = LOGP_INVALID;
  int c = c0 + threadIdx.x;
  for (; c + 3 * LOGP_THREADS < c1; c += 4 * LOGP_THREADS) {
    const i64 a0 = __ldg(x + c), a1 = __ldg(x + c + LOGP_THREADS), a2 = __ldg(x + c + 2 * LOGP_THREADS),
              a3 = __ldg(x + c + 3 * LOGP_THREADS);
    v = imax(imax(v, a0), imax(imax(a1, a2), a3));
  }
  for (; c < c1; c += LOGP_THREADS) v = imax(v, __ldg(x + c));
  v = block_max_i64(v, red);
  if (threadIdx.x == 0) pmax[(i64)row * nch + blockIdx.x] = v;
}

// One term e^(x - mx) at LSE_FE bits (rl.py:51-59): table entry of the clamped argument's top bits, interpolated on
// the s = fr - 12 low bits with a rounding shift. tab2[i] = (entry i, entry min(i + 1, last)): the two entries of an
// interpolation come with one 16-byte gather (the table is 2.6 MB, so most gathers go to L2 and their count is what
// the pass is bound by).
__device__ __forceinline__ i64 lse_term(i64 x, i64 mx, const longlong2* __restrict__ tab2, int fr) {
  const int s = fr - LSE_STEP;
  const i64 zc = imax(x - mx, -((i64)(-LSE_MIN) << fr));
  const i64 zi = zc >> s;
  const i64 r = zc - shl(zi, s);
  const longlong2 ab = __ldg(tab2 + (int)(zi + LSE_LAST));
  return ab.x + (((ab.y - ab.x) * r + ((i64)1 << (s - 1))) >> s);
}

// tab2[i] = (tab[i], tab[min(i + 1, n - 1)]).
__global__ void logp_pair_table_kernel(const i64* __restrict__ tab, longlong2* __restrict__ tab2, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) tab2[i] = make_longlong2(tab[i], tab[min(i + 1, n - 1)]);
}

// grid (nch, M): psum[row * nch + chunk] = sum of the chunk's terms against the row maximum: rowmax[row] when given,
// else the maximum of the row's nch_max chunk maxima in pmax (which it also leaves in rowmax_out[row], chunk 0).
__global__ void __launch_bounds__(LOGP_THREADS) logp_sum_kernel(const i64* __restrict__ lg, i64 ld,
                                                                 const i64* __restrict__ rowmax,
                                                                 const i64* __restrict__ pmax, int nch_max,
                                                                 i64* __restrict__ rowmax_out,
                                                                 const longlong2* __restrict__ tab, i64* __restrict__ psum,
                                                                 int V, int ch, int nch, int fr) {
  __shared__ i64 red[LOGP_THREADS / 32];
  const int row = blockIdx.y, c0 = blockIdx.x * ch, c1 = min(c0 + ch, V);
  i64 mx;
  if (rowmax) {
    mx = __ldg(rowmax + row);
  } else {
    i64 v = LOGP_INVALID;
    for (int j = threadIdx.x; j < nch_max; j += LOGP_THREADS) v = imax(v, pmax[(i64)row * nch_max + j]);
    mx = block_max_i64(v, red);
    if (blockIdx.x == 0 && threadIdx.x == 0) rowmax_out[row] = mx;
    __syncthreads();                                       // red is reused below
  }
  const i64* x = lg + (i64)row * ld;
  i64 acc = 0;
  int c = c0 + threadIdx.x;
  constexpr int U = 8;                                     // gathers in flight per thread: the pass is latency bound
  for (; c + (U - 1) * LOGP_THREADS < c1; c += U * LOGP_THREADS) {
    i64 a[U];
#pragma unroll
    for (int k = 0; k < U; ++k) a[k] = __ldg(x + c + k * LOGP_THREADS);
#pragma unroll
    for (int k = 0; k < U; ++k) a[k] = lse_term(a[k], mx, tab, fr);
#pragma unroll
    for (int k = 0; k < U; ++k) acc += a[k];
  }
  for (; c < c1; c += LOGP_THREADS) acc += lse_term(__ldg(x + c), mx, tab, fr);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    i64 t = 0;
#pragma unroll
    for (int w = 0; w < LOGP_THREADS / 32; ++w) t += red[w];
    psum[(i64)row * nch + blockIdx.x] = t;
  }
}

// One thread per row: out[row] = the maximum (sum = 0) or the sum (sum = 1) of the row's n partial values.
__global__ void logp_rowfold_kernel(const i64* __restrict__ part, int n, i64* __restrict__ out, int M, int sum) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  i64 v = part[(i64)row * n];
  for (int j = 1; j < n; ++j) {
    const i64 p = part[(i64)row * n + j];
    v = sum ? v + p : imax(v, p);
  }
  out[row] = v;
}

// One thread per row: S = the sum of nsum partial sums (or S itself, nsum = 1); the target term zt[row] when given,
// else logits[row, tok[row]] - rowmax[row]; out = (max(zt, -2^36) << (40 - fr)) - (ln S - 44 ln 2) (rl.py:61-65).
// A token outside [0, V) (a target term equal to the most negative int64), or a sum below 1, gives the most negative
// int64.
__global__ void logp_finish_kernel(const i64* __restrict__ psum, int nsum, const i64* __restrict__ zt,
                                   const i64* __restrict__ lg, i64 ld, const i64* __restrict__ tok,
                                   const i64* rowmax, const i64* __restrict__ lnt, i64* out, int M, int V, int fr) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  i64 S = 0;
  for (int j = 0; j < nsum; ++j) S += psum[(i64)row * nsum + j];
  i64 z;
  bool ok = S >= 1;
  if (zt) {
    z = zt[row];
    ok = ok && z != LOGP_INVALID;                          // no shard held the token
  } else {
    const i64 t = tok[row];
    ok = ok && t >= 0 && t < V;
    z = ok ? lg[(i64)row * ld + t] - rowmax[row] : 0;
  }
  if (!ok) {
    out[row] = LOGP_INVALID;
    return;
  }
  const i64 lse = ln_q(S, lnt) - (i64)LSE_FE * LN2Q;
  out[row] = shl(imax(z, -((i64)1 << 36)), FLN - fr) - lse;
}

}  // namespace bx
