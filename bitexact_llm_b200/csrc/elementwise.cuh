// Row-local integer stages between the linears of exact mode: RMSNorm + quantisation, RoPE + per-head
// quantisation + KV limb store, attention output division, SiLU * up + quantisation.
// One CTA per row (or per token and KV head); row maxima and sums are exact integer reductions (warp shuffles,
// then shared memory), so the thread count cannot change a bit. Bound violations set the sticky flag word.
//
// Same integers as src/bitexact/exact/segs.py:49-128 and the fused kernels of
// src/bitexact/vllm_plugin/exact_fuse.py:136-334.
#pragma once

#include <cooperative_groups.h>

#include "bx_rules.cuh"

namespace bx {

// ---- exact division helpers ----
// floor(x / d) and remainder for 0 <= x < 2^63 from inv = floor((2^64 - 1) / d): one high multiply, one fix-up.
__device__ __forceinline__ u64 uqr_recip(u64 x, u64 d, u64 inv, u64& rem) {
  u64 q = __umul64hi(x, inv);
  u64 r = x - q * d;
  if (r >= d) { q += 1; r -= d; }
  rem = r;
  return q;
}

// div_round (exact/ops.py:37-57) with the row-constant divisor r given with its reciprocal.
template <int NIT>
__device__ __forceinline__ i64 div_round_recip(i64 a, i64 p, u64 r, u64 inv) {
  u64 rem;
  const u64 mag = (u64)iabs(a);
  const u64 q0 = uqr_recip(mag, r, inv, rem);
  i64 Q, R;
  if (a < 0) { Q = -(i64)q0 - (rem != 0 ? 1 : 0); R = rem != 0 ? (i64)(r - rem) : 0; }
  else { Q = (i64)q0; R = (i64)rem; }
  i64 left = imax(p, 0);
#pragma unroll
  for (int i = 0; i < NIT; ++i) {
    if (left > 0) {                                    // a step with nothing left to shift in would change nothing
      const int c = (int)imin(left, 28);
      const u64 q1 = uqr_recip((u64)R << c, r, inv, rem);
      Q = shl(Q, c) + (i64)q1;
      R = (i64)rem;
      left -= c;
    }
  }
  if (p >= 0) return Q + (2 * R >= (i64)r ? 1 : 0);
  const int k = (int)iclamp(-p, 1, 62);
  return (Q + (1ll << (k - 1))) >> k;
}

// floor(num / den) for 0 <= num < 2^62 and 2^31 <= den <= 2^33 (quotient below 2^31): float64 estimate, exact integer
// fix-up. The conversion of num loses at most 2^8, i.e. 2^-23 of a quotient unit, and the division rounds by less
// than 2^-22, so the truncated estimate is the floor or one off; one correction each way settles it.
__device__ __forceinline__ i64 fdiv_pos_est(i64 num, i64 den) {
  i64 q = (i64)((double)num / (double)den);
  i64 r = num - q * den;
  if (r < 0) { q -= 1; r += den; }
  if (r >= den) { q += 1; }
  return q;
}

// ---- block reductions (exact, order free) ----
__device__ __forceinline__ i64 warp_max(i64 v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = imax(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ i64 warp_sum(i64 v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// All threads of the CTA get the result. `buf` holds 33 i64 in shared memory.
template <bool IS_MAX>
__device__ __forceinline__ i64 block_reduce(i64 v, i64* buf) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();                       // buf may still be read from a previous reduction
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  if (warp == 0) {
    i64 t = lane < nw ? buf[lane] : (IS_MAX ? (i64)0x8000000000000000ull : 0);
    t = IS_MAX ? warp_max(t) : warp_sum(t);
    if (lane == 0) buf[32] = t;
  }
  __syncthreads();
  return buf[32];
}

// 2^-t at out_bits for t >= 0 at 26 fractional bits: table 2^-f at 2^60 (step 2^-14) + linear interpolation
// (exact/ops.py:108-116).
template <bool SMEM_TABLE = false>
__device__ __forceinline__ i64 exp2neg_lut(i64 t, const i64* __restrict__ lut, int out_bits) {
  const i64 n = t >> FT2;
  const i64 f = t & ((1ll << FT2) - 1);
  const int idx = (int)(f >> (FT2 - EXP2_BITS));
  const i64 rr = f & ((1ll << (FT2 - EXP2_BITS)) - 1);
  const i64 a = SMEM_TABLE ? lut[idx] : __ldg(lut + idx);
  const i64 b = SMEM_TABLE ? lut[idx + 1] : __ldg(lut + idx + 1);
  const i64 v = a + rshs<FT2 - EXP2_BITS>((b - a) * rr);
  return rshc(v, (i64)(EXP2_ONE - out_bits) + n);
}

// Activation row -> limb planes a8[l][row][col] (optional), one element.
__device__ __forceinline__ void store_limb_planes(int8_t* a8, int64_t plane, int64_t off, int q) {
  int r = q;
  a8[off] = (int8_t)split8(r);
  a8[plane + off] = (int8_t)split8(r);
  a8[2 * plane + off] = (int8_t)split8(r);
}

// ---- RMSNorm + quant (segs.add_y + norm_q; exact_fuse._norm_kernel) ----
// MODE 0: x = emb[ids[row]] (int32 table); 1: x = xin + yin; 2: x = xin.
constexpr int NORM_THREADS = 256;
constexpr int NORM_EPT = 16;     // D <= 4096

// NT threads per row, EPT = ceil(D / NT) elements per thread (NT = 512, EPT = 4 for D = 2048: the row's serial
// instruction stream, not bandwidth, bounds this kernel at decode batch sizes).
template <int MODE, int NT, int EPT>
__global__ void __launch_bounds__(NT)
norm_kernel(const void* __restrict__ xin, const i64* __restrict__ yin, const i64* __restrict__ ids,
            const i64* __restrict__ gm, const i64* __restrict__ ge, i64* __restrict__ xo, int32_t* __restrict__ q,
            i64* __restrict__ sh_out, int8_t* __restrict__ a8, int32_t* flag, int M, int D, int lg, int do_norm) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  i64 x[EPT];
  i64 gmr[EPT], ger[EPT];          // gamma, loaded up front: their latency overlaps the row's loads and reductions
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * NT;
    gmr[k] = (do_norm && c < D) ? __ldg(gm + c) : 0;
    ger[k] = (do_norm && c < D) ? __ldg(ge + c) : 0;
  }
  i64 ax = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * NT;
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
  if (threadIdx.x == 0 && ax >= (1ll << 40)) *flag = 1;
  if (!do_norm) return;
  // rms (exact/ops.py:92-105)
  const i64 amax = imax(ax, 1);
  const i64 shx = imax((i64)bitlen(amax) - 25, -6);
  i64 S = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const i64 xs = rshc(x[k], shx);
    S += xs * xs;
  }
  S = block_reduce<false>(S, red);
  const i64 T = S + rshc(EPS60 * D, 60 - 2 * (FR - shx));
  const i64 m = (62 + lg - (i64)bitlen(T)) >> 1;
  const i64 s = 2 * m - lg;
  const i64 V = s >= 0 ? (s >= 64 ? 0 : shl(T, (int)s)) : (T >> (int)imin(-s, 63));
  const i64 r = isqrt(V);
  const i64 er = shx - FR - m;
  const u64 inv = ~0ull / (u64)r;
  // ndiv + quant(., -FN)
  i64 pmax = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * NT;
    if (c < D) {
      x[k] = div_round_recip<3>(x[k] * gmr[k], ger[k] - FR - er + FN, (u64)r, inv);
      pmax = imax(pmax, iabs(x[k]));
    }
  }
  pmax = block_reduce<true>(pmax, red);
  const i64 sh = quant_sh(pmax, -FN);
  if (threadIdx.x == 0) sh_out[row] = sh;
  const int64_t plane = (int64_t)M * D;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * NT;
    if (c < D) {
      const int qv = (int)rshc(x[k], sh + FN);
      q[row * D + c] = qv;
      if (a8) store_limb_planes(a8, plane, row * D + c, qv);
    }
  }
}

// ---- RoPE + per-head q quant + K / V limb store (segs.rope_y + q_group + tri_paged.store; _qkv_kernel) ----
// One CTA per (token, KV head); G query heads, head_dim HD (HD / 2 threads, each owning one rotation pair).
struct QkvParams {
  const i64* y;        // [N, (H + 2 HKV) HD] at FR
  const i64* cos;      // [max_pos, HD / 2] at 30 bits
  const i64* sin;
  const i64* pos;      // [N]
  const i64* slot;     // [N] flat cache slot, < 0: not stored (may be null with cache null)
  int8_t* cache;       // limb planes [nb, HKV, bs, 8 HD] or null
  int64_t sc_nb, sc_h, sc_bs;
  int bs;
  int32_t* q;          // [N, H HD]
  i64* sh;             // [N, H]
  int32_t* flag;
  int H, HKV, HD;
};

__global__ void qkv_kernel(const QkvParams p) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const int h = blockIdx.y;
  const int HH = p.HD / 2;
  const int G = p.H / p.HKV;
  const int dd = threadIdx.x;              // 0 .. HH-1
  const int64_t NT = (int64_t)(p.H + 2 * p.HKV) * p.HD;
  const i64 pos = p.pos[row];
  const i64* yr = p.y + row * NT;
  // Everything the thread reads is requested before the first use: the row's q / k / v values and the slot are in
  // flight together with the position and the rotation pair that depends on it (the kernel is a latency chain).
  constexpr int GPRE = 8;
  i64 xa[GPRE], xb[GPRE];
#pragma unroll
  for (int g = 0; g < GPRE; ++g) {
    xa[g] = 0;
    xb[g] = 0;
    if (g < G) {
      const int64_t qc = (int64_t)(h * G + g) * p.HD + dd;
      xa[g] = yr[qc];
      xb[g] = yr[qc + HH];
    }
  }
  const int64_t kc = (int64_t)p.H * p.HD + (int64_t)h * p.HD + dd;
  const int64_t vc = (int64_t)(p.H + p.HKV) * p.HD + (int64_t)h * p.HD + dd;
  const i64 k1 = yr[kc], k2 = yr[kc + HH];
  const i64 v1r = yr[vc], v2r = yr[vc + HH];
  const i64 slot = p.cache ? p.slot[row] : -1;
  const i64 cs = p.cos[pos * HH + dd];
  const i64 sn = p.sin[pos * HH + dd];
  i64 big = 0;
  i64 shmax = NEG_BIG;
  auto head = [&](int g, i64 x1, i64 x2) {
    const int64_t qc = (int64_t)(h * G + g) * p.HD + dd;
    big = imax(big, imax(iabs(x1), iabs(x2)));
    const i64 p1 = x1 * cs - x2 * sn;
    const i64 p2 = x2 * cs + x1 * sn;
    const i64 amax = block_reduce<true>(imax(iabs(p1), iabs(p2)), red);
    const i64 sh = quant_sh(amax, -(FR + FT));
    shmax = imax(shmax, sh);
    int32_t* qo = p.q + row * ((int64_t)p.H * p.HD) + qc;
    qo[0] = (int32_t)rshc(p1, sh + (FR + FT));
    qo[HH] = (int32_t)rshc(p2, sh + (FR + FT));
    if (threadIdx.x == 0) p.sh[row * p.H + h * G + g] = sh;
  };
#pragma unroll
  for (int g = 0; g < GPRE; ++g)
    if (g < G) head(g, xa[g], xb[g]);                   // G is the same for every thread of the grid
  for (int g = GPRE; g < G; ++g) {
    const int64_t qc = (int64_t)(h * G + g) * p.HD + dd;
    head(g, yr[qc], yr[qc + HH]);
  }
  big = imax(big, imax(imax(iabs(k1), iabs(k2)), imax(iabs(v1r), iabs(v2r))));
  const i64 k1o = rshs<FR + FT - FK>(k1 * cs - k2 * sn);
  const i64 k2o = rshs<FR + FT - FK>(k2 * cs + k1 * sn);
  const i64 v1 = rshs<FR - FV>(v1r);
  const i64 v2 = rshs<FR - FV>(v2r);
  const i64 kvbig = imax(imax(iabs(k1o), iabs(k2o)), imax(iabs(v1), iabs(v2)));
  big = block_reduce<true>(big, red);
  const i64 kvmax = block_reduce<true>(kvbig, red);
  if (threadIdx.x == 0 && (big >= (1ll << 31) || kvmax > LIM3 || shmax > FK + 3 - FZ)) *p.flag = 1;
  if (p.cache) {
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

// K / V int64 [N, HKV, HD] -> limb planes at flat slots (tri_paged.store, src/bitexact/vllm_plugin/tri_paged.py:311-335).
__global__ void kv_store_kernel(int8_t* cache, const i64* __restrict__ slot, const i64* __restrict__ k,
                                const i64* __restrict__ v, int64_t skz, int64_t skh, int64_t svz, int64_t svh,
                                int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, int HD) {
  const int64_t n = blockIdx.x;
  const int h = blockIdx.y;
  const i64 s = slot[n];
  if (s < 0) return;
  int8_t* base = cache + (s / bs) * sc_nb + (int64_t)h * sc_h + (s % bs) * sc_bs;
  for (int dd = threadIdx.x; dd < HD; dd += blockDim.x) {
    int kk = (int)k[n * skz + h * skh + dd], vv = (int)v[n * svz + h * svh + dd];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      base[i * HD + dd] = (int8_t)split8(kk);
      base[(3 + i) * HD + dd] = (int8_t)split8(vv);
    }
  }
}

// ---- attention output: o = div_round(num, 5, den), quant(o, -FR) (segs.attn_div + quant; _attn_out_kernel) ----
constexpr int AO_THREADS = 512;  // a row is a latency chain: more threads, fewer serial divisions each
constexpr int AO_EPT = 8;      // H * HD <= 4096
constexpr int AO_MAXH = 64;

__global__ void __launch_bounds__(AO_THREADS)
attn_out_kernel(const i64* __restrict__ num, const i64* __restrict__ den, int32_t* __restrict__ q,
                i64* __restrict__ sh_out, int8_t* __restrict__ a8, int M, int K2, int HD) {
  __shared__ i64 red[33];
  __shared__ u64 dens[AO_MAXH], invs[AO_MAXH];
  const int64_t row = blockIdx.x;
  const int nh = K2 / HD;
  i64 o[AO_EPT];
#pragma unroll
  for (int k = 0; k < AO_EPT; ++k) {                  // the numerators are in flight while the reciprocals are made
    const int c = threadIdx.x + k * AO_THREADS;
    o[k] = c < K2 ? num[row * K2 + c] : 0;
  }
  if (threadIdx.x < nh) {
    const u64 dv = (u64)den[row * nh + threadIdx.x];
    dens[threadIdx.x] = dv;
    invs[threadIdx.x] = dv ? ~0ull / dv : 0;
  }
  __syncthreads();
  i64 omax = 0;
#pragma unroll
  for (int k = 0; k < AO_EPT; ++k) {
    const int c = threadIdx.x + k * AO_THREADS;
    if (c < K2) {
      const int hd = c / HD;
      o[k] = dens[hd] ? div_round_recip<1>(o[k], FR - FV, dens[hd], invs[hd]) : 0;
      omax = imax(omax, iabs(o[k]));
    }
  }
  omax = block_reduce<true>(omax, red);
  const i64 sh = quant_sh(omax, -FR);
  if (threadIdx.x == 0) sh_out[row] = sh;
  const int64_t plane = (int64_t)M * K2;
#pragma unroll
  for (int k = 0; k < AO_EPT; ++k) {
    const int c = threadIdx.x + k * AO_THREADS;
    if (c < K2) {
      const int qv = (int)rshc(o[k], sh + FR);
      q[row * K2 + c] = qv;
      if (a8) store_limb_planes(a8, plane, row * K2 + c, qv);
    }
  }
}

// ---- SiLU(g) * u + quant(., -2 FR) (segs.silu_y + quant_silu; exact/ops.py:119-130; _silu_kernel) ----
constexpr int SILU_THREADS = 512;

template <bool SMEM_TABLE = false>
__device__ __forceinline__ i64 silu_p(i64 g, i64 u, const i64* __restrict__ lut, bool& bad) {
  const i64 a = imin(iabs(g), 64ll << FR);                       // <= 2^30: the product below is 32 x 32 -> 64 bits
  const i64 t = rshs<FR + 30 - FT2>((i64)((u64)(uint32_t)a * (u64)(uint32_t)L2E30));
  const i64 E = exp2neg_lut<SMEM_TABLE>(t, lut, 30);
  const i64 den = (1ll << 30) + E;
  const i64 nume = g >= 0 ? (1ll << 60) : shl(E, 30);
  const i64 sig = fdiv_pos_est(2 * nume + den, 2 * den);          // rdiv
  const i64 gc = iclamp(g, -(1ll << 32), 1ll << 32);
  const i64 s = rshs<30>(gc * sig);
  const u64 as = (u64)iabs(s), au = (u64)iabs(u);
  bad = iabs(g) > (1ll << 32);
  if ((as | au) >> 31) bad |= bitlen((i64)as) + bitlen((i64)au) > 62;      // both below 2^31: 62 bits cannot be passed
  return (i64)((u64)s * (u64)u);
}

template <int EPT>
__global__ void __launch_bounds__(SILU_THREADS)
silu_kernel(const i64* __restrict__ y, const i64* __restrict__ lut, int32_t* __restrict__ q, i64* __restrict__ sh_out,
            int8_t* __restrict__ a8, int32_t* flag, int M, int FF) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const i64* yr = y + row * (2 * (int64_t)FF);
  i64 P[EPT];
  i64 pmax = 0;
  bool anybad = false;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * SILU_THREADS;
    P[k] = 0;
    if (c < FF) {
      bool bad;
      P[k] = silu_p(yr[c], yr[FF + c], lut, bad);
      anybad |= bad;
      pmax = imax(pmax, iabs(P[k]));
    }
  }
  if (anybad) *flag = 1;
  pmax = block_reduce<true>(pmax, red);
  const i64 sh = quant_sh(pmax, -2 * FR);
  if (threadIdx.x == 0) sh_out[row] = sh;
  const int64_t plane = (int64_t)M * FF;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = threadIdx.x + k * SILU_THREADS;
    if (c < FF) {
      const int qv = (int)rshc(P[k], sh + 2 * FR);
      q[row * FF + c] = qv;
      if (a8) store_limb_planes(a8, plane, row * FF + c, qv);
    }
  }
}

// Cluster form of silu_kernel for decode batches: the FF columns of a row are split over the CTAs of a thread-block
// cluster (4 x 256 threads), the row maximum is exchanged through distributed shared memory. Four times as many
// CTAs as rows keep every SM busy when the batch has only a few hundred rows.
constexpr int SILU_CL = 4;
constexpr int SILU_CL_THREADS = 256;

template <int EPT>
__global__ void __launch_bounds__(SILU_CL_THREADS)
silu_cluster_kernel(const i64* __restrict__ y, const i64* __restrict__ lut, int32_t* __restrict__ q,
                    i64* __restrict__ sh_out, int8_t* __restrict__ a8, int32_t* flag, int M, int FF) {
  namespace cg = cooperative_groups;
  __shared__ i64 red[33];
  __shared__ i64 cta_max;
  cg::cluster_group cluster = cg::this_cluster();
  const int part = (int)cluster.block_rank();
  const int64_t row = blockIdx.x / SILU_CL;
  const int c0 = part * (FF / SILU_CL);
  const i64* yr = y + row * (2 * (int64_t)FF);
  i64 P[EPT];
  i64 pmax = 0;
  bool anybad = false;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = c0 + threadIdx.x + k * SILU_CL_THREADS;
    bool bad;
    P[k] = silu_p(yr[c], yr[FF + c], lut, bad);
    anybad |= bad;
    pmax = imax(pmax, iabs(P[k]));
  }
  if (anybad) *flag = 1;
  pmax = block_reduce<true>(pmax, red);
  if (threadIdx.x == 0) cta_max = pmax;
  cluster.sync();
  i64 rmax = 0;
#pragma unroll
  for (int r = 0; r < SILU_CL; ++r) rmax = imax(rmax, *cluster.map_shared_rank(&cta_max, r));
  const i64 sh = quant_sh(rmax, -2 * FR);
  if (part == 0 && threadIdx.x == 0) sh_out[row] = sh;
  const int64_t plane = (int64_t)M * FF;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int c = c0 + threadIdx.x + k * SILU_CL_THREADS;
    const int qv = (int)rshc(P[k], sh + 2 * FR);
    q[row * FF + c] = qv;
    if (a8) store_limb_planes(a8, plane, row * FF + c, qv);
  }
  cluster.sync();                                   // peers may still be reading cta_max
}

// Persistent form of silu_kernel with the 2^-f table (131 KB) in shared memory: one 1024-thread CTA per SM walks the
// rows. The table gathers are what the other forms wait for (they miss L1); from shared memory they cost a few
// cycles, and a CTA fetches the table once for all its rows.
constexpr int SILU_P_THREADS = 1024;
constexpr int SILU_TABLE = (1 << EXP2_BITS) + 1;

template <int EPT>
__global__ void __launch_bounds__(SILU_P_THREADS, 1)
silu_persistent_kernel(const i64* __restrict__ y, const i64* __restrict__ lut, int32_t* __restrict__ q,
                       i64* __restrict__ sh_out, int8_t* __restrict__ a8, int32_t* flag, int M, int FF) {
  extern __shared__ __align__(16) uint8_t silu_smem[];
  i64* tab = reinterpret_cast<i64*>(silu_smem);
  __shared__ i64 red[33];
  for (int i = threadIdx.x; i < SILU_TABLE; i += SILU_P_THREADS) tab[i] = __ldg(lut + i);
  __syncthreads();
  const int64_t plane = (int64_t)M * FF;
  bool anybad = false;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const i64* yr = y + row * (2 * (int64_t)FF);
    i64 P[EPT];
    i64 pmax = 0;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const int c = threadIdx.x + k * SILU_P_THREADS;
      P[k] = 0;
      if (c < FF) {
        bool bad;
        P[k] = silu_p<true>(yr[c], yr[FF + c], tab, bad);
        anybad |= bad;
        pmax = imax(pmax, iabs(P[k]));
      }
    }
    pmax = block_reduce<true>(pmax, red);
    const i64 sh = quant_sh(pmax, -2 * FR);
    if (threadIdx.x == 0) sh_out[row] = sh;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const int c = threadIdx.x + k * SILU_P_THREADS;
      if (c < FF) {
        const int qv = (int)rshc(P[k], sh + 2 * FR);
        q[row * FF + c] = qv;
        if (a8) store_limb_planes(a8, plane, row * FF + c, qv);
      }
    }
  }
  if (anybad) *flag = 1;
}

// ---- SiLU * up + quant in two kernels, for a gate / up projection sharded by output column over several GPUs ----
// silu_prod_kernel: y [N, 2 FFl] (the rank's gate columns, then its up columns) -> P int64 [N, FFl] and the row maximum
// of |P| over the rank's columns. The ranks then take the integer maximum of the row maxima (an exact all-reduce) and
// quant_rows_kernel quantises every shard with the same row exponent: the integers of silu_kernel on the full row.
template <int NT>
__global__ void __launch_bounds__(NT)
silu_prod_kernel(const i64* __restrict__ y, const i64* __restrict__ lut, i64* __restrict__ P, i64* __restrict__ rowmax,
                 int32_t* flag, int FFl) {
  __shared__ i64 red[33];
  const int64_t row = blockIdx.x;
  const i64* yr = y + row * (2 * (int64_t)FFl);
  i64 pmax = 0;
  bool anybad = false;
  for (int c = threadIdx.x; c < FFl; c += NT) {
    bool bad;
    const i64 v = silu_p(yr[c], yr[FFl + c], lut, bad);
    anybad |= bad;
    pmax = imax(pmax, iabs(v));
    P[row * FFl + c] = v;
  }
  if (anybad) *flag = 1;
  pmax = block_reduce<true>(pmax, red);
  if (threadIdx.x == 0) rowmax[row] = pmax;
}

// q = rshc(P, sh + fbits) with sh = quant_sh(rowmax, -fbits) (exact/ops.py:82-89); also the limb planes of q (optional)
// with row pitch `ldq` and plane size `plane` elements, so that a rank can write its columns into the full-width planes.
__global__ void __launch_bounds__(256)
quant_rows_kernel(const i64* __restrict__ P, const i64* __restrict__ rowmax, int fbits, int32_t* __restrict__ q,
                  int64_t ldq, i64* __restrict__ sh_out, int8_t* __restrict__ a8, int64_t plane, int K) {
  const int64_t row = blockIdx.x;
  const i64 sh = quant_sh(rowmax[row], -(i64)fbits);
  if (threadIdx.x == 0 && sh_out) sh_out[row] = sh;
  for (int c = threadIdx.x; c < K; c += 256) {
    const int qv = (int)rshc(P[row * K + c], sh + fbits);
    q[row * ldq + c] = qv;
    if (a8) store_limb_planes(a8, plane, row * ldq + c, qv);
  }
}

}  // namespace bx
