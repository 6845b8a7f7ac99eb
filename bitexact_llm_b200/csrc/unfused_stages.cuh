// The element-wise stages of the reference's STANDALONE exact engine as kernels of their own
// (src/bitexact/exact/segs.py:44-128, src/bitexact/exact/ops.py:92-143): rms, ndiv, row maxima for quant, RoPE
// without the quantisation, softmax weights of a dense score matrix, the attention division. The serving path fuses
// them (elementwise.cuh, paged_attention.cuh); these exist so that code written against `bitexact.exact.segs` /
// `bitexact.exact.ops` keeps running, stage by stage, with the same integers. One CTA per row, rows of any length.
#pragma once

#include "elementwise.cuh"
#include "paged_attention.cuh"

namespace bx {

constexpr int US_THREADS = 256;

// ops.rms: (r, er) with sqrt(mean(x^2) + 1e-5) = r 2^er, 2^30 <= r < 2^31; amax[row] = max |x| (for the 2^40 bound).
__global__ void __launch_bounds__(US_THREADS)
rms_kernel(const i64* __restrict__ x, i64* __restrict__ r_out, i64* __restrict__ er_out, i64* __restrict__ amax_out,
           int D, int lg) {
  __shared__ i64 red[33];
  const i64* xr = x + (int64_t)blockIdx.x * D;
  i64 ax = 0;
  for (int c = threadIdx.x; c < D; c += US_THREADS) ax = imax(ax, iabs(xr[c]));
  ax = block_reduce<true>(ax, red);
  const i64 amax = imax(ax, 1);
  const i64 shx = imax((i64)bitlen(amax) - 25, -6);
  i64 S = 0;
  for (int c = threadIdx.x; c < D; c += US_THREADS) {
    const i64 xs = rshc(xr[c], shx);
    S += xs * xs;
  }
  S = block_reduce<false>(S, red);
  if (threadIdx.x == 0) {
    const i64 T = S + rshc(EPS60 * D, 60 - 2 * (FR - shx));
    const i64 m = (62 + lg - (i64)bitlen(T)) >> 1;
    const i64 s = 2 * m - lg;
    const i64 V = s >= 0 ? (s >= 64 ? 0 : shl(T, (int)s)) : (T >> (int)imin(-s, 63));
    r_out[blockIdx.x] = isqrt(V);
    er_out[blockIdx.x] = shx - FR - m;
    if (amax_out) amax_out[blockIdx.x] = ax;
  }
}

// segs.ndiv: P = div_round(x gamma_m, gamma_e - FR - er + FN, r), one rounding per element.
__global__ void __launch_bounds__(US_THREADS)
ndiv_kernel(const i64* __restrict__ x, const i64* __restrict__ gm, const i64* __restrict__ ge,
            const i64* __restrict__ r, const i64* __restrict__ er, i64* __restrict__ P, int D) {
  const int64_t row = blockIdx.x;
  const i64 rr = r[row], e = er[row];
  for (int c = threadIdx.x; c < D; c += US_THREADS)
    P[row * D + c] = div_round<3>(x[row * D + c] * gm[c], ge[c] - FR - e + FN, rr);
}

// max |P| per row (the first half of ops.quant; bx_exact_quant_rows is the second).
__global__ void __launch_bounds__(US_THREADS)
rowmax_abs_kernel(const i64* __restrict__ P, i64* __restrict__ rowmax, int K) {
  __shared__ i64 red[33];
  const i64* pr = P + (int64_t)blockIdx.x * K;
  i64 ax = 0;
  for (int c = threadIdx.x; c < K; c += US_THREADS) ax = imax(ax, iabs(pr[c]));
  ax = block_reduce<true>(ax, red);
  if (threadIdx.x == 0) rowmax[blockIdx.x] = ax;
}

// segs.rope_y without the reshapes: y [N, (H + 2 HKV) HD] at FR -> Pq int64 [N, H, HD] (at FR + FT, unquantised),
// k int64 [N, HKV, HD] at FK, v int64 [N, HKV, HD] at FV. One CTA per token.
__global__ void __launch_bounds__(US_THREADS)
rope_kernel(const i64* __restrict__ y, const i64* __restrict__ cos, const i64* __restrict__ sin,
            const i64* __restrict__ pos, i64* __restrict__ Pq, i64* __restrict__ k, i64* __restrict__ v, int H, int HKV,
            int HD) {
  const int64_t n = blockIdx.x;
  const int half = HD / 2;
  const i64* yr = y + n * (int64_t)(H + 2 * HKV) * HD;
  const i64* c = cos + pos[n] * half;
  const i64* s = sin + pos[n] * half;
  for (int e = threadIdx.x; e < (H + HKV) * half; e += US_THREADS) {
    const int hd = e / half, d = e % half;
    const i64 x1 = yr[hd * HD + d], x2 = yr[hd * HD + half + d];
    const i64 a = x1 * c[d] - x2 * s[d], b = x2 * c[d] + x1 * s[d];
    if (hd < H) {
      Pq[(n * H + hd) * HD + d] = a;
      Pq[(n * H + hd) * HD + half + d] = b;
    } else {
      const int hk = hd - H;
      k[(n * HKV + hk) * HD + d] = rshc(a, FR + FT - FK);
      k[(n * HKV + hk) * HD + half + d] = rshc(b, FR + FT - FK);
    }
  }
  for (int e = threadIdx.x; e < HKV * HD; e += US_THREADS)
    v[n * HKV * HD + e] = rshc(yr[(int64_t)(H + HKV) * HD + e], FR - FV);
}

// ops.softmax_w (exact rule, or the int8 rule with ptab) of one row of scores: key s takes part iff ok[row, s]
// (when ok is given) or s <= qpos[row]; masked weights are 0. p int32 [R, S], den int64 [R].
__global__ void __launch_bounds__(US_THREADS)
softmax_w_kernel(const i64* __restrict__ raw, const uint8_t* __restrict__ ok, const i64* __restrict__ qpos,
                 const i64* __restrict__ sh, AttnParams w, int32_t* __restrict__ p, i64* __restrict__ den, int S) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const i64* rr = raw + row * S;
  const uint8_t* okr = ok ? ok + row * S : nullptr;
  const i64 qp = qpos ? qpos[row] : (i64)S;
  i64 mx = ATT_NEG;
  for (int s = threadIdx.x; s < S; s += US_THREADS)
    if (okr ? okr[s] != 0 : s <= qp) mx = imax(mx, rr[s]);
  mx = block_reduce<true>(mx, red);
  const i64 rowshift = sh ? (i64)(FK + 3 - FZ) - sh[row] : 0;
  i64 sum = 0;
  for (int s = threadIdx.x; s < S; s += US_THREADS) {
    i64 pv = 0;
    if (okr ? okr[s] != 0 : s <= qp) pv = attn_weight_any(w, rr[s], mx, rowshift);
    p[row * S + s] = (int32_t)pv;
    sum += pv;
  }
  sum = block_reduce<false>(sum, red);
  if (threadIdx.x == 0) den[row] = sum;
}

// segs.attn_div without the reshapes: o[z, d] = div_round(num[z, d], FR - FV, den[z]).
__global__ void __launch_bounds__(US_THREADS)
attn_div_kernel(const i64* __restrict__ num, const i64* __restrict__ den, i64* __restrict__ o, int HD) {
  const int64_t z = blockIdx.x;
  const i64 dn = den[z];
  for (int d = threadIdx.x; d < HD; d += US_THREADS) o[z * HD + d] = dn ? div_round<3>(num[z * HD + d], FR - FV, dn) : 0;
}

}  // namespace bx
