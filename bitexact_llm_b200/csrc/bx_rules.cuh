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

// Per-tile scalars held across the lanes of a warp: slot s of lane l holds the value of tile row (or column)
// 32 s + l. A warp loads them once per tile, before it waits for the accumulators, and hands a value round by
// shuffle when an output needs it: no global load remains between the accumulator read-out and the stores.
template <int NS>
__device__ __forceinline__ i64 lane_slot(const i64 (&v)[NS], int idx) {
  i64 x = v[0];
#pragma unroll
  for (int s = 1; s < NS; ++s)
    if ((idx >> 5) == s) x = v[s];
  return x;
}
template <int NS>
__device__ __forceinline__ int lane_slot(const int (&v)[NS], int idx) {
  int x = v[0];
#pragma unroll
  for (int s = 1; s < NS; ++s)
    if ((idx >> 5) == s) x = v[s];
  return x;
}

// a0 + a1 2^8 + a2 2^16 + a3 2^24 + a4 2^32 of five signed 32-bit accumulators, as three widening multiply-adds.
__device__ __forceinline__ i64 join5(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4) {
  i64 t = (i64)(int32_t)a0;
  asm("mad.wide.s32 %0, %1, 256, %0;" : "+l"(t) : "r"(a1));
  asm("mad.wide.s32 %0, %1, 65536, %0;" : "+l"(t) : "r"(a2));
  asm("mad.wide.s32 %0, %1, 16777216, %0;" : "+l"(t) : "r"(a3));
  return t + (i64)((u64)a4 << 32);
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

// round_shift_hl for a whole warp (all 32 lanes call it together; lanes with on = false take no part in the result).
// When every lane that is on shifts right by k = -p = 1 .. 31 bits with k >= d, |T| < 2^61 and |B| < 2^60, the short
// form is taken: nothing wraps, H 2^32 + L is V = T 2^d + B exactly, and the two-word result
// (H << (32 - k)) + ((L + 2^(k-1)) >> k) is floor((V + 2^(k-1)) / 2^k). With X = B + 2^(k-1) = Xh 2^d + Xl
// (0 <= Xl < 2^d) that is floor((T + Xh + Xl / 2^d) / 2^(k-d)) = (T + Xh) >> (k - d): the fraction Xl / 2^d < 1
// cannot carry into the floor. |H| < 2^(29+d) + 2^28 < 2^(31+k) and |y| < 2^62, so the flag stays clear. Same
// integers as round_shift_hl at a fifth of its instructions; any other case takes round_shift_hl itself.
__device__ __forceinline__ i64 round_rule_warp(i64 T, i64 B, int d, i64 p, bool on, bool& bad) {
  const bool in = p < 0 && p > -32 && -p >= (i64)d &&
                  (((u64)(T + (1ll << 61)) >> 62) | ((u64)(B + (1ll << 60)) >> 61)) == 0;
  if (__all_sync(0xffffffffu, !on || in)) {
    const int k = on ? (int)(-p) : 31;
    bad = false;
    return (T + ((B + (1ll << (k - 1))) >> d)) >> (k - d);
  }
  bad = false;
  if (!on) return 0;
  return round_shift_hl(T, B, d, p, bad);
}

}  // namespace bx
