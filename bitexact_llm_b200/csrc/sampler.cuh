// Integer sampler: greedy first-argmax, or Gumbel-max with integer Gumbel noise keyed by (seed, token index).
//
// The noise of a row is a pure function of its key: the raw 64-bit words of numpy's PCG64 stream
// default_rng([20261022, seed, t]) (one word per vocabulary entry), turned into -ln(-ln u) with integer
// arithmetic (ln table + linear interpolation). The token is the FIRST index of max(round(l td / tn) + g).
// Everything runs on the device: SeedSequence hashing, the 128-bit LCG (each thread jumps ahead to its own
// vocabulary run in O(log i) steps, then walks it), XSL-RR output, Gumbel, chunked (max, first index) pairs.
//
// Same integers as src/bitexact/sampling.py:27-67 (CPU) and as gpu_pcg.raw_rows + sample(gumbel(.))
// (src/bitexact/vllm_plugin/gpu_pcg.py:54-108, vllm_plugin/sampler.py:57-88).
#pragma once

#include "bx_rules.cuh"
#include "elementwise.cuh"

namespace bx {

constexpr u64 PCG_MULT_HI = 2549297995355413924ull;
constexpr u64 PCG_MULT_LO = 4865540595714422341ull;
constexpr i64 LN2Q = 762123384786ll;      // round(ln 2 * 2^40)
constexpr i64 UMIN = 9008;
constexpr int FLN = 40;
constexpr uint32_t SEED_BASE = 20261022u;
constexpr int SAMPLE_THREADS = 256;

struct u128 {
  u64 hi, lo;
};
__device__ __forceinline__ u128 mul128(u128 a, u128 b) {
  u128 r;
  r.lo = a.lo * b.lo;
  r.hi = __umul64hi(a.lo, b.lo) + a.hi * b.lo + a.lo * b.hi;
  return r;
}
__device__ __forceinline__ u128 add128(u128 a, u128 b) {
  u128 r;
  r.lo = a.lo + b.lo;
  r.hi = a.hi + b.hi + (r.lo < a.lo ? 1ull : 0ull);
  return r;
}

// numpy SeedSequence([SEED_BASE, seed, t]) -> PCG64 (state, inc) after seeding.
__device__ inline void pcg_seed(u64 seed, u64 t, u128& state, u128& inc) {
  const uint32_t MULT_A = 0x931E8875u, MULT_B = 0x58F38DEDu, MIX_L = 0xCA01F9DDu, MIX_R = 0x4973F715u;
  uint32_t ent[5];
  int n = 0;
  ent[n++] = SEED_BASE;
  ent[n++] = (uint32_t)seed;
  if (seed >> 32) ent[n++] = (uint32_t)(seed >> 32);
  ent[n++] = (uint32_t)t;
  if (t >> 32) ent[n++] = (uint32_t)(t >> 32);
  uint32_t hc = 0x43B0D7E5u;
  auto hashmix = [&](uint32_t v) {
    v ^= hc;
    hc *= MULT_A;
    v *= hc;
    return v ^ (v >> 16);
  };
  auto mix = [&](uint32_t x, uint32_t y) {
    uint32_t r = MIX_L * x - MIX_R * y;
    return r ^ (r >> 16);
  };
  uint32_t pool[4];
  for (int i = 0; i < 4; ++i) pool[i] = hashmix(i < n ? ent[i] : 0u);
  for (int s = 0; s < 4; ++s)
    for (int d = 0; d < 4; ++d)
      if (s != d) pool[d] = mix(pool[d], hashmix(pool[s]));
  for (int s = 4; s < n; ++s)
    for (int d = 0; d < 4; ++d) pool[d] = mix(pool[d], hashmix(ent[s]));
  uint32_t hb = 0x8B51F9DDu, w[8];
  for (int i = 0; i < 8; ++i) {
    uint32_t v = pool[i & 3] ^ hb;
    hb *= MULT_B;
    v *= hb;
    w[i] = v ^ (v >> 16);
  }
  const u64 u0 = (u64)w[0] | ((u64)w[1] << 32), u1 = (u64)w[2] | ((u64)w[3] << 32);
  const u64 u2 = (u64)w[4] | ((u64)w[5] << 32), u3 = (u64)w[6] | ((u64)w[7] << 32);
  const u128 initstate = {u0, u1}, initseq = {u2, u3};
  inc.hi = (initseq.hi << 1) | (initseq.lo >> 63);
  inc.lo = (initseq.lo << 1) | 1ull;
  const u128 mult = {PCG_MULT_HI, PCG_MULT_LO};
  state = add128(inc, initstate);
  state = add128(mul128(state, mult), inc);
}

// state after `delta` further LCG steps.
__device__ inline u128 pcg_advance(u128 state, u128 inc, u64 delta) {
  u128 cur_mult = {PCG_MULT_HI, PCG_MULT_LO}, cur_plus = inc;
  u128 acc_mult = {0, 1}, acc_plus = {0, 0};
  while (delta) {
    if (delta & 1) {
      acc_mult = mul128(acc_mult, cur_mult);
      acc_plus = add128(mul128(acc_plus, cur_mult), cur_plus);
    }
    cur_plus = mul128(add128(cur_mult, u128{0, 1}), cur_plus);
    cur_mult = mul128(cur_mult, cur_mult);
    delta >>= 1;
  }
  return add128(mul128(acc_mult, state), acc_plus);
}

// (mult, plus) of `delta` LCG steps at once: state -> mult * state + plus.
__device__ inline void pcg_jump(u128 inc, u64 delta, u128& mult, u128& plus) {
  u128 cur_mult = {PCG_MULT_HI, PCG_MULT_LO}, cur_plus = inc;
  mult = u128{0, 1};
  plus = u128{0, 0};
  while (delta) {
    if (delta & 1) {
      mult = mul128(mult, cur_mult);
      plus = add128(mul128(plus, cur_mult), cur_plus);
    }
    cur_plus = mul128(add128(cur_mult, u128{0, 1}), cur_plus);
    cur_mult = mul128(cur_mult, cur_mult);
    delta >>= 1;
  }
}

// XSL-RR output of a state.
__device__ __forceinline__ u64 pcg_output(u128 state) {
  const u64 x = state.hi ^ state.lo;
  const int rot = (int)(state.hi >> 58);
  return (x >> rot) | (x << ((64 - rot) & 63));
}

__device__ __forceinline__ u64 pcg_next(u128& state, u128 inc) {
  state = add128(mul128(state, u128{PCG_MULT_HI, PCG_MULT_LO}), inc);
  const u64 x = state.hi ^ state.lo;
  const int rot = (int)(state.hi >> 58);
  return (x >> rot) | (x << ((64 - rot) & 63));
}

// ln(n) at 40 bits for n >= 1 (sampling.py:40-47).
__device__ __forceinline__ i64 ln_q(i64 n, const i64* __restrict__ lnt) {
  const int k = bitlen(n) - 1;
  const i64 m = k <= 52 ? shl(n, 52 - k) : (n >> (k - 52));
  const int idx = (int)((m >> 36) - (1 << 16));
  const i64 r = (m >> 16) & ((1 << 20) - 1);
  const i64 a = __ldg(lnt + idx);
  return (i64)k * LN2Q + a + (((__ldg(lnt + idx + 1) - a) * r) >> 20);
}

// -ln(-ln u) at `bits` fractional bits (sampling.py:50-59).
__device__ __forceinline__ i64 gumbel_q(i64 raw, const i64* __restrict__ lnt, int bits) {
  const i64 U = iclamp((raw >> 11) & ((1ll << 53) - 1), UMIN, (1ll << 53) - UMIN);
  const i64 Dd = (1ll << 53) - U;
  i64 lna;
  if (Dd < (1ll << 45)) {
    const i64 dq = Dd >> 13;
    const i64 e = dq >> 8;
    lna = ln_q(Dd, lnt) - 53 * LN2Q + (dq >> 1) + (5 * e * e) / (24ll << 24);
  } else {
    const i64 A = 53 * LN2Q - ln_q(U, lnt);
    lna = ln_q(imax(A, 1), lnt) - FLN * LN2Q;
  }
  const int s = FLN - bits;
  return s > 0 ? ((-lna + (1ll << (s - 1))) >> s) : shl(-lna, -s);
}

// Raw words only: keys int64 [n, 2] (seed, t) -> out int64 [n, V]  (gpu_pcg.raw_rows).
__global__ void __launch_bounds__(SAMPLE_THREADS)
pcg_raw_kernel(const i64* __restrict__ keys, i64* __restrict__ out, int V, int run) {
  const int64_t row = blockIdx.y;
  const int64_t e0 = ((int64_t)blockIdx.x * SAMPLE_THREADS + threadIdx.x) * run;
  if (e0 >= V) return;
  u128 st, inc;
  pcg_seed((u64)keys[2 * row], (u64)keys[2 * row + 1], st, inc);
  st = pcg_advance(st, inc, (u64)e0);
  const int64_t e1 = e0 + run < V ? e0 + run : V;
  for (int64_t e = e0; e < e1; ++e) out[row * V + e] = (i64)pcg_next(st, inc);
}

// The generator state after numpy's seeding, as gpu_pcg.seed_state lays it out: st int64 [n, 4] = state hi, state lo,
// increment hi, increment lo.
__global__ void pcg_seed_state_kernel(const i64* __restrict__ keys, i64* __restrict__ st, int n) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  u128 state, inc;
  pcg_seed((u64)keys[2 * r], (u64)keys[2 * r + 1], state, inc);
  st[4 * r] = (i64)state.hi;
  st[4 * r + 1] = (i64)state.lo;
  st[4 * r + 2] = (i64)inc.hi;
  st[4 * r + 3] = (i64)inc.lo;
}

// Raw words from given generator states (gpu_pcg.raw_from_state): st int64 [n, 4] -> out int64 [n, V].
__global__ void __launch_bounds__(SAMPLE_THREADS)
pcg_raw_state_kernel(const i64* __restrict__ stv, i64* __restrict__ out, int V, int run) {
  const int64_t row = blockIdx.y;
  const int64_t e0 = ((int64_t)blockIdx.x * SAMPLE_THREADS + threadIdx.x) * run;
  if (e0 >= V) return;
  u128 st, inc;
  st.hi = (u64)stv[4 * row];
  st.lo = (u64)stv[4 * row + 1];
  inc.hi = (u64)stv[4 * row + 2];
  inc.lo = (u64)stv[4 * row + 3];
  st = pcg_advance(st, inc, (u64)e0);
  const int64_t e1 = e0 + run < V ? e0 + run : V;
  for (int64_t e = e0; e < e1; ++e) out[row * V + e] = (i64)pcg_next(st, inc);
}

// Chunked sampling pass. rows: int64 [M, 4] = seed, t, tn, td (tn == 0: greedy). Each CTA handles vocabulary
// entries [chunk * ch, chunk * ch + ch) of one row and writes its (max value, first index) pair.
// Thread t takes entries c0 + t, c0 + t + 256, ...: a warp reads 32 consecutive logits, and the generator of the
// thread jumps 256 states per entry (one 128-bit multiply-add, the cost of a single step).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_part_kernel(const i64* __restrict__ logits, int64_t ld, const i64* __restrict__ rows,
                   const i64* __restrict__ lnt, i64* __restrict__ pmax, i64* __restrict__ pidx, int V, int ch,
                   int nch, int bits, i64 voff) {
  __shared__ i64 smax[SAMPLE_THREADS / 32], sidx[SAMPLE_THREADS / 32];
  __shared__ i64 gtab[41];
  const int64_t row = blockIdx.y;
  const int chunk = blockIdx.x;
  const i64 tn = rows[4 * row + 2], td = rows[4 * row + 3];
  const int64_t c0 = (int64_t)chunk * ch;
  const int64_t c1 = c0 + ch < V ? c0 + ch : V;
  const int64_t e0 = c0 + threadIdx.x;
  i64 best = (i64)0x8000000000000000ull, bidx = 0x7fffffffffffffffll;
  const i64* lr = logits + row * ld;     // local columns; vocabulary index = voff + column
  if (tn == 0) {
    for (int64_t e = e0; e < c1; e += SAMPLE_THREADS) {
      const i64 v = lr[e];
      if (v > best) { best = v; bidx = voff + e; }
    }
  } else {
    // Exact pruning. The noise g is a non-decreasing function of the uniform U within each branch of gumbel_q, so
    // for 1 - u in (2^-j, 2^-(j-1)] it is at most gtab[j] = g at 1 - u = 2^-j (taken with the same function). An
    // entry whose scaled logit plus that bound stays below a value some entry of the row already reached cannot be
    // the first maximum; only the others (a few per cent) pay for the two table logarithms and the division.
    // The bound every lane prunes with is the warp's best value, refreshed every fourth entry; the comparison is
    // strict, so equal values (which the first-index rule must see) are always evaluated.
    if (threadIdx.x >= 1 && threadIdx.x <= 40) {
      const u64 t = (1ull << 53) - (1ull << (53 - threadIdx.x));
      gtab[threadIdx.x] = gumbel_q((i64)(t << 11), lnt, bits);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    u128 st, inc, jm, jp;
    pcg_seed((u64)rows[4 * row], (u64)rows[4 * row + 1], st, inc);
    st = pcg_advance(st, inc, (u64)(voff + e0) + 1);           // the state whose output is the word of entry e0
    pcg_jump(inc, SAMPLE_THREADS, jm, jp);
    const u64 dv = (u64)(2 * tn);
    const u64 inv = ~0ull / dv;
    const bool prunable = dv < (1ull << 31);
    i64 wb = (i64)0x8000000000000000ull;
    // Four entries per round: their logits are loaded first (independent loads in flight), then each is processed.
    for (int64_t eb = c0 + (threadIdx.x & ~31); eb < c1; eb += 4 * SAMPLE_THREADS) {
      i64 lg[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t e = eb + lane + (int64_t)k * SAMPLE_THREADS;
        lg[k] = e < c1 ? lr[e] : 0;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t e = eb + lane + (int64_t)k * SAMPLE_THREADS;
        if (eb + (int64_t)k * SAMPLE_THREADS >= c1) break;       // warp-uniform
        const bool act = e < c1;
        const u64 w = pcg_output(st);
        st = add128(mul128(jm, st), jp);
        const i64 U = iclamp((i64)((w >> 11) & ((1ull << 53) - 1)), UMIN, (1ll << 53) - UMIN);
        const int j = __clzll((1ll << 53) - U) - 10;           // 1 - u in (2^-j, 2^-(j-1)], 1 <= j <= 40
        // rdiv(l * td, tn) = floor((2 l td + tn) / (2 tn))
        const i64 a = 2 * lg[k] * td + tn;
        bool pass = act;
        const i64 lb = imax(best, wb);
        if (act && prunable && lb > -(1ll << 61)) {
          const i64 m = lb - gtab[j];                          // floor(a / dv) + gtab[j] < lb  <=>  a < m dv
          if (m > -(1ll << 31) && m < (1ll << 31)) pass = !(a < m * (i64)dv);
        }
        if (__any_sync(0xffffffffu, pass)) {
          if (pass) {
            const i64 g = gumbel_q((i64)w, lnt, bits);
            u64 rem;
            const u64 qd = uqr_recip((u64)iabs(a), dv, inv, rem);
            const i64 fq = a < 0 ? -(i64)qd - (rem != 0 ? 1 : 0) : (i64)qd;
            const i64 v = fq + g;
            if (v > best) { best = v; bidx = voff + e; }
          }
        }
      }
      wb = warp_max(best);
    }
  }
  // first index of the maximum: larger value wins, then the smaller index
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const i64 ov = __shfl_xor_sync(0xffffffffu, best, o);
    const i64 oi = __shfl_xor_sync(0xffffffffu, bidx, o);
    if (ov > best || (ov == best && oi < bidx)) { best = ov; bidx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { smax[warp] = best; sidx[warp] = bidx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
      if (smax[w] > best || (smax[w] == best && sidx[w] < bidx)) { best = smax[w]; bidx = sidx[w]; }
    pmax[row * nch + chunk] = best;
    pidx[row * nch + chunk] = bidx;
  }
}

// tok[row] = first index of the maximum over the chunks; omax (may be null) receives the maximum itself.
__global__ void sample_combine_kernel(const i64* __restrict__ pmax, const i64* __restrict__ pidx,
                                      i64* __restrict__ tok, i64* __restrict__ omax, int M, int nch) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  i64 best = pmax[(int64_t)row * nch], bidx = pidx[(int64_t)row * nch];
  for (int c = 1; c < nch; ++c) {
    const i64 v = pmax[(int64_t)row * nch + c], i = pidx[(int64_t)row * nch + c];
    if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
  }
  tok[row] = bidx;
  if (omax) omax[row] = best;
}

}  // namespace bx
