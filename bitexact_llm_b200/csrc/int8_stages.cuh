// Row-local integer stages of int8 mode between its linears: RMSNorm + 2-limb row quantisation, RoPE + KV limb
// store, attention output division, SiLU-table * up + quantisation. They consume the int64 output y of the fused
// int8 linear (post already applied) and emit the next linear's input: activation limb planes int8 [2, M, K]
// (limb i of row m at row i * M + m, the layout of the reference's stack_limbs) and the row scale (mant, e).
//
// Same integers as src/bitexact/int8/ops.py:24-108 and int8/segs.py:48-118, and as the fused kernels of
// src/bitexact/vllm_plugin/tri_fuse.py:82-265 and vllm_plugin/tri_mlp.py:86-150.
#pragma once

#include "bx_rules.cuh"
#include "elementwise.cuh"
#include "int8_linear.cuh"

namespace bx {
namespace i8 {

constexpr int FR = 16, FG = 12, FA = 12, FT = 16, FQ = 14, FV = 14;
constexpr i64 EPS40 = 10995116;
constexpr i64 QMAX2 = 127 << 8;
constexpr i64 SILU_LO = -(32 << 12), SILU_HI = 32 << 12;

// floor(n / d) for d > 0 from inv = floor((2^64 - 1) / d), |n| < 2^63.
__device__ __forceinline__ i64 fdiv_recip(i64 n, u64 d, u64 inv) {
  u64 rem;
  const u64 q = uqr_recip((u64)iabs(n), d, inv, rem);
  return n < 0 ? -(i64)q - (rem != 0 ? 1 : 0) : (i64)q;
}

// quant_rows(z, 2) pieces from the row's max |z| (int8/ops.py:24-35): shift sh, scaled maximum as_.
__device__ __forceinline__ void quant_scale(i64 zmax, i64& sh, i64& as_) {
  const i64 amax = imax(zmax, 1);
  sh = (i64)bitlen(amax) - 30;
  as_ = rsh_t(amax, sh);
}
__device__ __forceinline__ int quant2(i64 z, i64 sh, i64 as_, u64 inv) {
  const i64 zs = rsh_t(z, sh);
  return (int)fdiv_recip(2 * (zs * QMAX2) + as_, (u64)(2 * as_), inv);     // rdiv(zs * qmax, as_)
}
__device__ __forceinline__ void store_limbs2(int8_t* a8, int64_t plane, int64_t off, int q) {
  const int lo = ((q + 128) & 255) - 128;
  a8[off] = (int8_t)lo;
  a8[plane + off] = (int8_t)((q - lo) >> 8);
}
// norm24 (int8/ops.py:70-73)
__device__ __forceinline__ void norm24(i64 mant, i64 e, i64& m_out, i64& e_out) {
  const i64 b = (i64)bitlen(mant) - 24;
  m_out = rsh_t(mant, b);
  e_out = e + b;
}

// MODE 0: x = emb[ids]; 1: x = xin + yin; 2: x = xin. With do_norm: pre_norm(x, gamma) (int8/segs.py:48-53).
template <int MODE>
__global__ void __launch_bounds__(NORM_THREADS)
int8_norm_kernel(const void* __restrict__ xin, const i64* __restrict__ yin, const i64* __restrict__ ids,
                 const i64* __restrict__ gamma, i64* __restrict__ xo, int8_t* __restrict__ a8, i64* __restrict__ mant,
                 i64* __restrict__ eo, int32_t* flag, int M, int D, int do_norm) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  i64 x[NORM_EPT];
  i64 ax = 0;
#pragma unroll
  for (int k = 0; k < NORM_EPT; ++k) {
    const int c = threadIdx.x + k * NORM_THREADS;
    x[k] = 0;
    if (c < D) {
      if (MODE == 0) x[k] = (i64) reinterpret_cast<const int32_t*>(xin)[ids[row] * D + c];
      else if (MODE == 1) x[k] = reinterpret_cast<const i64*>(xin)[row * D + c] + yin[row * D + c];
      else x[k] = reinterpret_cast<const i64*>(xin)[row * D + c];
      if (xo) xo[row * D + c] = x[k];
      ax = imax(ax, iabs(x[k]));
    }
  }
  ax = block_reduce<true>(ax, red);
  if (!do_norm) {
    if (threadIdx.x == 0 && ax >= (1ll << 42)) *flag = 1;
    return;
  }
  const i64 shx = (i64)bitlen(imax(ax, 1)) - 24;                       // rms (int8/ops.py:76-84)
  i64 S = 0, zmax = 0;
#pragma unroll
  for (int k = 0; k < NORM_EPT; ++k) {
    const int c = threadIdx.x + k * NORM_THREADS;
    if (c < D) {
      const i64 xs = rsh_t(x[k], shx);
      S += xs * xs;
      x[k] = x[k] * gamma[c];
      zmax = imax(zmax, iabs(x[k]));
    }
  }
  S = block_reduce<false>(S, red);
  zmax = block_reduce<true>(zmax, red);
  const i64 r = isqrt(S / D + rsh_t(EPS40, 40 - 2 * (FR - shx)));
  i64 sh, as_;
  quant_scale(zmax, sh, as_);
  const u64 inv = ~0ull / (u64)(2 * as_);
  const int64_t plane = (int64_t)M * D;
#pragma unroll
  for (int k = 0; k < NORM_EPT; ++k) {
    const int c = threadIdx.x + k * NORM_THREADS;
    if (c < D) store_limbs2(a8, plane, row * D + c, quant2(x[k], sh, as_, inv));
  }
  if (threadIdx.x == 0) {
    const i64 mq = fdiv(2 * shl(as_, 30) + r, 2 * r);                  // rdiv(as_ << 30, r)
    norm24(mq, sh - FG - shx - 30, mant[row], eo[row]);
  }
}

// RoPE (16-bit cos / sin) of q and k, v >> 2, bound flag, K / V limb planes stored in the paged cache
// (int8/segs.py:69-88; tri_fuse._qkv_kernel). One CTA per (token, KV head), HD / 2 threads.
struct Qkv8Params {
  const i64* y;
  const i64* cos;
  const i64* sin;
  const i64* pos;
  const i64* slot;
  int8_t* cache;
  int64_t sc_nb, sc_h, sc_bs;
  int bs;
  i64* q64;          // [N, HKV, G, HD] (may be null)
  int32_t* q32;      // same values as int32 (may be null)
  int32_t* flag;
  int H, HKV, HD;
};

__global__ void int8_qkv_kernel(const Qkv8Params p) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const int h = blockIdx.y;
  const int HH = p.HD / 2, G = p.H / p.HKV, dd = threadIdx.x;
  const int64_t NT = (int64_t)(p.H + 2 * p.HKV) * p.HD;
  constexpr int SHR = FT + FR - FQ;
  const i64 pos = p.pos[row];
  const i64 cs = p.cos[pos * HH + dd], sn = p.sin[pos * HH + dd];
  const i64* yr = p.y + row * NT;
  i64 big = 0;
  for (int g = 0; g < G; ++g) {
    const int64_t qc = (int64_t)(h * G + g) * p.HD + dd;
    const i64 x1 = yr[qc], x2 = yr[qc + HH];
    const i64 q1 = rshs<SHR>(x1 * cs - x2 * sn), q2 = rshs<SHR>(x2 * cs + x1 * sn);
    big = imax(big, imax(iabs(q1), iabs(q2)));
    const int64_t qo = row * ((int64_t)p.H * p.HD) + qc;            // [N, HKV, G, HD] == [N, H, HD]
    if (p.q64) { p.q64[qo] = q1; p.q64[qo + HH] = q2; }
    if (p.q32) { p.q32[qo] = (int32_t)q1; p.q32[qo + HH] = (int32_t)q2; }
  }
  const int64_t kc = (int64_t)p.H * p.HD + (int64_t)h * p.HD + dd;
  const int64_t vc = (int64_t)(p.H + p.HKV) * p.HD + (int64_t)h * p.HD + dd;
  const i64 k1 = yr[kc], k2 = yr[kc + HH];
  const i64 k1o = rshs<SHR>(k1 * cs - k2 * sn), k2o = rshs<SHR>(k2 * cs + k1 * sn);
  const i64 v1 = rshs<FR - FV>(yr[vc]), v2 = rshs<FR - FV>(yr[vc + HH]);
  big = imax(big, imax(imax(iabs(k1o), iabs(k2o)), imax(iabs(v1), iabs(v2))));
  big = block_reduce<true>(big, red);
  if (threadIdx.x == 0 && big > LIM3) *p.flag = 1;
  if (p.cache) {
    const i64 slot = p.slot[row];
    if (slot >= 0) {
      int8_t* base = p.cache + (slot / p.bs) * p.sc_nb + (int64_t)h * p.sc_h + (slot % p.bs) * p.sc_bs;
      int kk1 = (int)k1o, kk2 = (int)k2o, vv1 = (int)v1, vv2 = (int)v2;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        base[i * p.HD + dd] = (int8_t)split8(kk1);
        base[i * p.HD + HH + dd] = (int8_t)split8(kk2);
        base[(3 + i) * p.HD + dd] = (int8_t)split8(vv1);
        base[(3 + i) * p.HD + HH + dd] = (int8_t)split8(vv2);
      }
    }
  }
}

// o = rdiv(num << 2, den) per head, then pre_plain(o) (int8/segs.py:101-109; tri_fuse._attn_out_kernel).
__global__ void __launch_bounds__(AO_THREADS)
int8_attn_out_kernel(const i64* __restrict__ num, const i64* __restrict__ den, int8_t* __restrict__ a8,
                     i64* __restrict__ mant, i64* __restrict__ eo, int M, int K2, int HD) {
  __shared__ i64 red[33];
  __shared__ u64 dens[AO_MAXH], invs[AO_MAXH];
  const int64_t row = blockIdx.x;
  const int nh = K2 / HD;
  if (threadIdx.x < nh) {
    const u64 dv = 2 * (u64)den[row * nh + threadIdx.x];
    dens[threadIdx.x] = dv;
    invs[threadIdx.x] = dv ? ~0ull / dv : 0;
  }
  __syncthreads();
  i64 o[AO_EPT];
  i64 omax = 0;
#pragma unroll
  for (int k = 0; k < AO_EPT; ++k) {
    const int c = threadIdx.x + k * AO_THREADS;
    o[k] = 0;
    if (c < K2) {
      const int hd = c / HD;
      if (dens[hd]) o[k] = fdiv_recip(2 * shl(num[row * K2 + c], FR - FV) + (i64)(dens[hd] >> 1), dens[hd], invs[hd]);
      omax = imax(omax, iabs(o[k]));
    }
  }
  omax = block_reduce<true>(omax, red);
  i64 sh, as_;
  quant_scale(omax, sh, as_);
  const u64 inv = ~0ull / (u64)(2 * as_);
  const int64_t plane = (int64_t)M * K2;
#pragma unroll
  for (int k = 0; k < AO_EPT; ++k) {
    const int c = threadIdx.x + k * AO_THREADS;
    if (c < K2) store_limbs2(a8, plane, row * K2 + c, quant2(o[k], sh, as_, inv));
  }
  if (threadIdx.x == 0) norm24(as_, sh - FR, mant[row], eo[row]);
}

// SiLU at FR from the table at step 2^-12 with linear interpolation (int8/ops.py:100-108).
__device__ __forceinline__ i64 silu_tab(i64 g, const i64* __restrict__ lut) {
  const i64 gi = g >> (FR - FA);
  const i64 r = g - shl(gi, FR - FA);
  const i64 i = iclamp(gi, SILU_LO, SILU_HI - 1) - SILU_LO;
  const i64 a = __ldg(lut + i);
  const i64 v = a + rshs<FR - FA>((__ldg(lut + i + 1) - a) * r);
  return gi >= SILU_HI ? g : (gi < SILU_LO ? 0 : v);
}

// h = rsh(silu(g) * u, FR), pre_plain(h); the row maxima of |silu(g)| and |u| go to scr[0], scr[1] as atomic
// maxima (int8/segs.py:111-118; tri_mlp._h_kernel / _quant_kernel with ATOMIC).
template <int EPT>
__global__ void __launch_bounds__(SILU_THREADS)
int8_silu_kernel(const i64* __restrict__ y, const i64* __restrict__ lut, int8_t* __restrict__ a8,
                 i64* __restrict__ mant, i64* __restrict__ eo, i64* __restrict__ scr, int M, int FF) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const i64* yr = y + row * (2 * (int64_t)FF);
  i64 hv[EPT];
  i64 hmax = 0, smax = 0, umax = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * SILU_THREADS;
    hv[k] = 0;
    if (c < FF) {
      const i64 sg = silu_tab(yr[c], lut), u = yr[FF + c];
      hv[k] = rshs<FR>((i64)((u64)sg * (u64)u));
      hmax = imax(hmax, iabs(hv[k]));
      smax = imax(smax, iabs(sg));
      umax = imax(umax, iabs(u));
    }
  }
  hmax = block_reduce<true>(hmax, red);
  smax = block_reduce<true>(smax, red);
  umax = block_reduce<true>(umax, red);
  if (threadIdx.x == 0 && scr) {
    atomicMax(reinterpret_cast<long long*>(scr), (long long)smax);
    atomicMax(reinterpret_cast<long long*>(scr + 1), (long long)umax);
  }
  i64 sh, as_;
  quant_scale(hmax, sh, as_);
  const u64 inv = ~0ull / (u64)(2 * as_);
  const int64_t plane = (int64_t)M * FF;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * SILU_THREADS;
    if (c < FF) store_limbs2(a8, plane, row * FF + c, quant2(hv[k], sh, as_, inv));
  }
  if (threadIdx.x == 0) norm24(as_, sh - FR, mant[row], eo[row]);
}

// segs.post on a raw int_mm output (src/bitexact/int8/segs.py:62-67): c int32 [R, N] with limb i of row m at row
// i * M + m -> y int64 [M, N]; flag when checked and some |t| >= 2^38.
__global__ void int8_post_kernel(const int32_t* __restrict__ c, const i64* __restrict__ mul, i64 fmsh,
                                 const i64* __restrict__ mant, const i64* __restrict__ e, i64* __restrict__ y,
                                 int32_t* flag, int M, int N, int checked) {
  const int64_t total = (int64_t)M * N;
  bool bad = false;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = t / N, n = t % N;
    const i64 acc = (i64)c[t] + shl((i64)c[total + t], 8);
    const i64 tv = rsh_t((i64)((u64)acc * (u64)mul[n]), fmsh);
    bad |= iabs(tv) >= (1ll << 38);
    y[t] = rsh_t((i64)((u64)tv * (u64)mant[m]), 8 - e[m]);
  }
  if (checked && bad) *flag = 1;
}

// segs.post on the joined accumulator acc = c0 + (c1 << 8) as int64 [M, N] (the form the reference's `post` takes).
__global__ void int8_post_acc_kernel(const i64* __restrict__ acc, const i64* __restrict__ mul, i64 fmsh,
                                     const i64* __restrict__ mant, const i64* __restrict__ e, i64* __restrict__ y,
                                     int32_t* flag, int M, int N, int checked) {
  const int64_t total = (int64_t)M * N;
  bool bad = false;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = t / N, n = t % N;
    const i64 tv = rsh_t((i64)((u64)acc[t] * (u64)mul[n]), fmsh);
    bad |= iabs(tv) >= (1ll << 38);
    y[t] = rsh_t((i64)((u64)tv * (u64)mant[m]), 8 - e[m]);
  }
  if (checked && bad) *flag = 1;
}

// The same in two steps, for a gate / up projection sharded by output column over several GPUs: step 1 on the
// rank's columns writes h and the row maxima of |h| (and the |silu(g)|, |u| maxima for the bound flag); the caller
// takes the integer maximum of the row maxima over the ranks; step 2 quantises the rank's columns with the scale of
// the FULL row. Same integers as int8_silu_kernel on the full row.
template <int EPT>
__global__ void __launch_bounds__(SILU_THREADS)
int8_silu_prod_kernel(const i64* __restrict__ y, const i64* __restrict__ lut, i64* __restrict__ h,
                      i64* __restrict__ rowmax, i64* __restrict__ scr, int M, int FF) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const i64* yr = y + row * (2 * (int64_t)FF);
  i64 hmax = 0, smax = 0, umax = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * SILU_THREADS;
    if (c < FF) {
      const i64 sg = silu_tab(yr[c], lut), u = yr[FF + c];
      const i64 hv = rshs<FR>((i64)((u64)sg * (u64)u));
      h[row * FF + c] = hv;
      hmax = imax(hmax, iabs(hv));
      smax = imax(smax, iabs(sg));
      umax = imax(umax, iabs(u));
    }
  }
  hmax = block_reduce<true>(hmax, red);
  smax = block_reduce<true>(smax, red);
  umax = block_reduce<true>(umax, red);
  if (threadIdx.x == 0) {
    rowmax[row] = hmax;
    if (scr) {
      atomicMax(reinterpret_cast<long long*>(scr), (long long)smax);
      atomicMax(reinterpret_cast<long long*>(scr + 1), (long long)umax);
    }
  }
}

// pre_plain of the rows of h [M, K] given the maxima of the full rows: limb planes a8 [2][M][K], mant, e.
__global__ void __launch_bounds__(256)
int8_quant_rows_kernel(const i64* __restrict__ h, const i64* __restrict__ rowmax, int8_t* __restrict__ a8,
                       i64* __restrict__ mant, i64* __restrict__ eo, int M, int K) {
  const int64_t row = blockIdx.x;
  i64 sh, as_;
  quant_scale(rowmax[row], sh, as_);
  const u64 inv = ~0ull / (u64)(2 * as_);
  const int64_t plane = (int64_t)M * K;
  for (int c = threadIdx.x; c < K; c += blockDim.x) store_limbs2(a8, plane, row * K + c, quant2(h[row * K + c], sh, as_, inv));
  if (threadIdx.x == 0 && mant) norm24(as_, sh - FR, mant[row], eo[row]);
}

// flag |= any layer's max|silu(g)| * max|u| >= 2^62 (int64 product, wrapping like the reference's), then reset
// (tri_fuse._flag_kernel, src/bitexact/vllm_plugin/tri_fuse.py:248-265).
__global__ void int8_flag_end_kernel(i64* scr, int32_t* flag, int L) {
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    const i64 s = scr[2 * i], u = scr[2 * i + 1];
    if ((i64)((u64)s * (u64)u) >= (1ll << 62)) *flag = 1;
    scr[2 * i] = 0;
    scr[2 * i + 1] = 0;
  }
}

}  // namespace i8
}  // namespace bx
