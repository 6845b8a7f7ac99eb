// Device-side integer rules of the bit-exact engine: round-half-up shifts, floor / rounding division,
// exact integer square root, bit length, signed base-256 limbs. Every function is a fixed rule on int64,
// so results do not depend on thread count, tiling or order. Left shifts are done on uint64 (two's-complement
// wrap, the behaviour of the reference's tensor shifts); right shifts of int64 are arithmetic.
//
// Reference: src/bitexact/intops.py:14-70 and src/bitexact/exact/ops.py:25-79.
#pragma once

#include <stdint.h>

namespace bx {

typedef long long i64;
typedef unsigned long long u64;

constexpr int FR = 24;    // residual stream, linear outputs, logits
constexpr int FT = 30;    // cos / sin
constexpr int FN = 40;    // normalised activations
constexpr int QB = 22;    // |q| <= 2^22
constexpr int FK = 17, FV = 19, FP = 22;
constexpr int FT2 = 26, FZ = 26;
constexpr int EXP2_BITS = 14, EXP2_ONE = 60;
constexpr i64 NEG_BIG = -(1ll << 20);
constexpr i64 LIM3 = 8355711;
constexpr i64 EPS60 = 11529215046068ll;
constexpr i64 L2E30 = 1549082005ll;

__device__ __forceinline__ i64 shl(i64 x, int s) { return (i64)((u64)x << s); }   // 0 <= s <= 63
__device__ __forceinline__ i64 imin(i64 a, i64 b) { return a < b ? a : b; }
__device__ __forceinline__ i64 imax(i64 a, i64 b) { return a > b ? a : b; }
__device__ __forceinline__ i64 iabs(i64 a) { return a < 0 ? -a : a; }
__device__ __forceinline__ i64 iclamp(i64 x, i64 lo, i64 hi) { return imin(imax(x, lo), hi); }

// Bits of x >= 0 (0 for 0).
__device__ __forceinline__ int bitlen(i64 x) { return 64 - __clzll(x); }

// round(x / 2^s) ties up for a compile-time s > 0.
template <int S>
__device__ __forceinline__ i64 rshs(i64 x) {
  return (x + (1ll << (S - 1))) >> S;
}

// round(x / 2^s) with the shift clamped to [-62, 62]; s <= 0 multiplies (exact/ops.py:25-34).
__device__ __forceinline__ i64 rshc(i64 x, i64 s) {
  int c = (int)iclamp(s, -62, 62);
  if (c > 0) return (x + (1ll << (c - 1))) >> c;
  return shl(x, -c);
}

// floor(a / b) for b > 0.
__device__ __forceinline__ i64 fdiv(i64 a, i64 b) {
  i64 q = a / b;
  return (a - q * b < 0) ? q - 1 : q;
}

// round(a / b) ties up for b > 0 (intops.py:42-44).
__device__ __forceinline__ i64 rdiv(i64 a, i64 b) { return fdiv(2 * a + b, 2 * b); }

// floor(sqrt(x)) for 0 <= x < 2^63: float64 estimate, then exact integer corrections (intops.py:46-52).
__device__ __forceinline__ i64 isqrt(i64 x) {
  i64 s = (i64)floor(sqrt((double)x));
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (s * s > x) s -= 1;
    if ((s + 1) * (s + 1) <= x) s += 1;
  }
  return s;
}

// round(a * 2^p / r) for |a| < 2^62, 2^11 <= r < 2^34: long division in NIT chunks of 28 bits
// (exact/ops.py:37-57; NIT = 3 is the general case, NIT = 1 is exact for 0 <= p <= 28).
template <int NIT>
__device__ __forceinline__ i64 div_round(i64 a, i64 p, i64 r) {
  i64 Q = fdiv(a, r);
  i64 R = a - Q * r;
  i64 left = imax(p, 0);
#pragma unroll
  for (int i = 0; i < NIT; ++i) {
    int c = (int)imin(left, 28);
    i64 X = shl(R, c);
    i64 q1 = X / r;                      // X >= 0
    Q = shl(Q, c) + q1;
    R = X - q1 * r;
    left -= c;
  }
  if (p >= 0) return Q + (2 * R >= r ? 1 : 0);
  int k = (int)iclamp(-p, 1, 62);
  return (Q + (1ll << (k - 1))) >> k;
}

// Row exponent of the power-of-two quantisation from the row's max |P| (exact/ops.py:82-89).
__device__ __forceinline__ i64 quant_sh(i64 amax, i64 eps) {
  i64 e = amax != 0 ? (i64)bitlen(amax) + eps : NEG_BIG;
  return imax(e - QB, NEG_BIG);
}

// One signed base-256 digit of r; r becomes the rest (intops.py:62-70).
__device__ __forceinline__ int split8(int& r) {
  int lo = ((r + 128) & 255) - 128;
  r = (r - lo) >> 8;
  return lo;
}

// round((T * 2^d + B) * 2^p) by the two-word rule (exact/ops.py:60-79), and whether bits were lost or the
// result left (-2^62, 2^62) (exact/wmm.py:143-149). 0 <= d <= 30.
__device__ __forceinline__ i64 round_shift_hl(i64 T, i64 B, int d, i64 p, bool& bad) {
  const int s = 32 - d;
  i64 H = T >> s;
  i64 L = shl(T & ((1ll << s) - 1), d) + B;
  H += L >> 32;
  L &= 0xFFFFFFFFll;
  i64 y;
  if (p >= 0) {
    const int pp = (int)imin(p, 30);
    y = shl(H, 32 + pp) + shl(L, pp);
    const i64 lim = 1ll << (31 - pp);
    bad = (H >= lim) | (H < -lim) | ((p > 30) & ((H != 0) | (L != 0)));
  } else {
    const i64 k = -p;
    if (k < 32) {
      const int k1 = (int)k;
      y = shl(H, 32 - k1) + ((L + (1ll << (k1 - 1))) >> k1);
      const i64 lim = 1ll << (31 + k1);
      bad = (H >= lim) | (H < -lim);
    } else {
      const int k2 = (int)imin(k, 94);
      const i64 carry = (k2 == 32) ? ((L + (1ll << 31)) >> 32) : (1ll << (k2 - 33));
      y = (H + carry) >> (k2 - 32);
      bad = false;
    }
  }
  bad = bad | (y <= -(1ll << 62)) | (y >= (1ll << 62));
  return y;
}

// round_shift_hl with a short cut for the common case. For a weight row on its own grid (d = 0) without residual
// entries (B = 0) and a shift of 1 .. 31 bits (p = -k), H 2^32 + L = T and the two-word rule
// (H << (32 - k)) + ((L + 2^(k-1)) >> k) is (T + 2^(k-1)) >> k, because H 2^32 is a multiple of 2^k. With
// |T| < 2^61 (|q| <= 2^22, |W| < 2^23, K < 43690) no bit can be lost and |y| < 2^62: the flag stays clear. Same
// integers as round_shift_hl, a fifth of its instructions.
__device__ __forceinline__ i64 exact_round(i64 T, i64 B, int d, i64 p, bool plain_row, bool& bad) {
  if (plain_row && p < 0 && p > -32) {
    const int k = (int)(-p);
    bad = false;
    return (T + (1ll << (k - 1))) >> k;
  }
  return round_shift_hl(T, B, d, p, bad);
}

}  // namespace bx
