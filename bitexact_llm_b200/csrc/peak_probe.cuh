// Measured int8 tensor-pipe peak: one CTA per SM issues tcgen05.mma kind::i8 (M = 128, N = 256, K = 32) back to back
// on operands that stay in shared memory, into two alternating TMEM accumulators. No TMA, no global loads and no
// epilogue inside the loop, so the rate is what the tensor pipe and its shared-memory operand path deliver: the
// denominator the limb-GEMM roofline fractions are quoted against.
#pragma once

#include "bx_ptx.cuh"

namespace bx {

constexpr int PEAK_N = 256;
constexpr int PEAK_SMEM = 200 * 1024;     // more than half of an SM's shared memory: one CTA per SM

struct PeakShared {
  uint64_t done;
  uint32_t tmem_base;
};

__global__ void __launch_bounds__(128, 1) i8_peak_kernel(int iters) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tile = base;                              // 128 rows x 128 bytes (four K slices), 128-byte swizzle
  uint8_t* b_tile = base + 128 * 128;                  // 256 rows x 128 bytes
  PeakShared* sh = reinterpret_cast<PeakShared*>(base + (128 + PEAK_N) * 128);
  // operand bytes: any non-trivial pattern (all-zero operands would draw less power than a real GEMM)
  for (int i = threadIdx.x; i < (128 + PEAK_N) * 128 / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(base)[i] = (uint32_t)i * 2654435761u + blockIdx.x;
  if (threadIdx.x == 0) {
    mbar_init(&sh->done, 1);
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (threadIdx.x < 32) {
    tmem_alloc(&sh->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_i8(PEAK_N);
    const uint32_t a0 = smem_u32(a_tile), b0 = smem_u32(b_tile);
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_i8(tmem + (i & 1) * PEAK_N, umma_desc_sw128(a0 + ks * 32), umma_desc_sw128(b0 + ks * 32), idesc,
                i >= 2 || ks > 0);
    }
    umma_commit(&sh->done);
    if (!mbar_wait(&sh->done, 0)) atomicAdd(&g_wait_timeouts, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace bx
