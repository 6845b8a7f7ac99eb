// The unfused entry points of the reference's standalone engine: the exact batched integer product `bmm`
// (src/bitexact/bmm.py:78-102) and the linear epilogue as a stage of its own, `segs.lin_y` on a dense product T
// and a residual B (src/bitexact/exact/segs.py:25-32, exact/wmm.py:132-150). The serving path never calls them
// (it uses the fused linear and the paged attention kernel); they exist so that code written against the
// reference's unfused API runs unchanged.
#pragma once

#include "bx_rules.cuh"

namespace bx {

// c[z, m, n] = sum_k a[z, m, k] * b[z, k, n], int64 wrap-free as long as the reference's bounds hold (operands of at
// most 3 limbs, K < 43690: |sum| < 2^62). One CTA per 32 x 32 output tile; operands staged through shared memory.
constexpr int BMM_T = 32;

template <typename TA, typename TB>
__global__ void __launch_bounds__(256)
bmm_kernel(const TA* __restrict__ a, const TB* __restrict__ b, i64* __restrict__ c, int M, int N, int K, int64_t saz,
           int64_t sam, int64_t sak, int64_t sbz, int64_t sbk, int64_t sbn) {
  __shared__ i64 As[BMM_T][BMM_T + 1];
  __shared__ i64 Bs[BMM_T][BMM_T + 1];
  const int z = blockIdx.z;
  const int m0 = blockIdx.y * BMM_T, n0 = blockIdx.x * BMM_T;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8 threads, 4 rows each
  i64 acc[4] = {0, 0, 0, 0};
  for (int k0 = 0; k0 < K; k0 += BMM_T) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i;
      const int m = m0 + r, ka = k0 + tx;
      As[r][tx] = (m < M && ka < K) ? (i64)a[z * saz + m * sam + ka * sak] : 0;
      const int kb = k0 + r, n = n0 + tx;
      Bs[r][tx] = (kb < K && n < N) ? (i64)b[z * sbz + kb * sbk + n * sbn] : 0;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < BMM_T; ++k) {
      const i64 bv = Bs[k][tx];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] += As[ty + 8 * i][k] * bv;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 8 * i, n = n0 + tx;
    if (m < M && n < N) c[((int64_t)z * M + m) * N + n] = acc[i];
  }
}

// y[m, n] = round((T[m, n] 2^d[n] + B[m, n]) 2^(sh[m] + g[n] - d[n] + FR)); B dense (may be null) or, when ec is
// given, the ELL residual gathered from q.
__global__ void __launch_bounds__(256)
epilogue_kernel(const i64* __restrict__ T, const i64* __restrict__ B, const int32_t* __restrict__ q, int64_t ldq,
                const int32_t* __restrict__ cnt, const int32_t* __restrict__ ec, const i64* __restrict__ ev, int R,
                const i64* __restrict__ d, const i64* __restrict__ g, const i64* __restrict__ sh, i64* __restrict__ y,
                int32_t* flag, int M, int N, int checked) {
  const int64_t total = (int64_t)M * N;
  bool any_bad = false;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = t / N;
    const int n = (int)(t % N);
    i64 Bv = B ? B[t] : 0;
    if (cnt) {
      const int c = cnt[n];
      for (int j = 0; j < c; ++j) Bv += (i64)q[m * ldq + ec[(int64_t)n * R + j]] * ev[(int64_t)n * R + j];
    }
    const int dn = (int)d[n];
    bool bad;
    y[t] = round_shift_hl(T[t], Bv, dn, sh[m] + g[n] - (i64)dn + FR, bad);
    any_bad |= bad;
  }
  if (checked && any_bad) *flag = 1;
}

}  // namespace bx
