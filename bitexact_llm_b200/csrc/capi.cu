// C ABI of libbitexact_b200.so (declared in include/bitexact_b200.h). One translation unit: the kernel headers
// are included here so that the device-side status word is shared by every kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>

#include "../../include/bitexact_b200.h"
#include "exact_linear.cuh"
#include "exact_linear_splitk.cuh"
#include "exact_linear_rows.cuh"
#include "int8_linear.cuh"
#include "int8_linear_splitk.cuh"
#include "int8_stages.cuh"
#include "elementwise.cuh"
#include "paged_attention.cuh"
#include "prefill_attention.cuh"
#include "sampler.cuh"
#include "logp.cuh"
#include "decompose.cuh"
#include "unfused.cuh"
#include "unfused_stages.cuh"
#include "peak_probe.cuh"
#include "bmm_limb.cuh"

namespace {

using namespace bx;

long long g_launches = 0;   // kernels launched through this library (host-side count)

// Host-side shadow of the device status word: non-zero once the host has SEEN a timed-out device-side wait
// (bx_device_status returned non-zero). Launching entry points then return BX_EDEVICE without
// launching, until bx_clear_device_status. Reading the device word itself needs a synchronising copy, which a
// launch path cannot afford; the engines' check() does that read.
std::atomic<int> g_status_seen{0};

inline int launched(int n) {
  if (cudaGetLastError() != cudaSuccess) return BX_ELAUNCH;
  g_launches += n;
  return BX_OK;
}

// Kernel attributes (opt-in dynamic shared memory) and device properties are per device: every cache of them is
// indexed by the ordinal of the current device. The flags are atomics so that concurrent first calls from several
// host threads are well defined (they would store the same value).
constexpr int BX_MAX_DEVICES = 64;

struct PerDevice {
  std::atomic<int> v[BX_MAX_DEVICES];
};

inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= BX_MAX_DEVICES) return -1;
  return dev;
}

// Runs `setup` (returns cudaError_t) once per device; BX_OK or BX_ELAUNCH.
template <class F>
inline int once_per_device(PerDevice& done, F&& setup) {
  const int dev = current_device();
  if (dev < 0) return BX_ELAUNCH;
  if (done.v[dev].load(std::memory_order_acquire)) return BX_OK;
  if (setup() != cudaSuccess) return BX_ELAUNCH;
  done.v[dev].store(1, std::memory_order_release);
  return BX_OK;
}

// Number of SMs of the current device (0 on error).
inline int device_sms() {
  static PerDevice sms;
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = sms.v[dev].load(std::memory_order_acquire);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
    sms.v[dev].store(n, std::memory_order_release);
  }
  return n;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// int8 [planes, rows, K] row-major -> 3-D map (K, rows, planes), box (128 bytes, box_rows, planes), 128B swizzle.
bool make_map(CUtensorMap* m, const void* base, uint64_t K, uint64_t rows, uint64_t planes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {K, rows, planes};
  cuuint64_t strides[2] = {K, rows * K};
  cuuint32_t box[3] = {128, box_rows, (cuuint32_t)planes};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The same tensor with boxes of `box_rows` rows of ONE plane (the B-operand chunks of the CTA-pair kernels).
bool make_map_chunks(CUtensorMap* m, const void* base, uint64_t K, uint64_t rows, uint64_t planes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {K, rows, planes};
  cuuint64_t strides[2] = {K, rows * K};
  cuuint32_t box[3] = {128, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int TA>
int launch_exact(const CUtensorMap& mw, const CUtensorMap& ma, const ExactEpiParams& ep, int K, cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  exact_linear_kernel<TA><<<m_tiles * n_tiles, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mw, ma, ep, K, m_tiles);
  return launched(1);
}

template <int TA>
int launch_exact_splitk(const CUtensorMap& mw, const CUtensorMap& ma, const ExactEpiParams& ep, int K, int split,
                        cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_splitk_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(m_tiles * n_tiles * split), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, exact_linear_splitk_kernel<TA>, mw, ma, ep, K, m_tiles) != cudaSuccess) return BX_ELAUNCH;
  return launched(1);
}

// Split-K with the activation rows as the 128-row operand (exact_linear_rows_splitk_kernel).
template <int TA>
int launch_exact_rows_splitk(const CUtensorMap& mact, const CUtensorMap& mwt, const ExactEpiParams& ep, int K, int split,
                             cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_rows_splitk_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int w_tiles = (ep.N + TA - 1) / TA;
  const int row_blocks = (ep.M + WROWS - 1) / WROWS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(w_tiles * row_blocks * split), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, exact_linear_rows_splitk_kernel<TA>, mact, mwt, ep, K, w_tiles) != cudaSuccess)
    return BX_ELAUNCH;
  return launched(1);
}

template <int TA>
int launch_exact_persistent(const CUtensorMap& mw, const CUtensorMap& ma, const ExactEpiParams& ep, int K,
                            cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_persistent_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int sms = device_sms();
  if (sms <= 0) return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  const int total = m_tiles * n_tiles;
  const int grid = total < sms ? total : sms;
  exact_linear_persistent_kernel<TA><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mw, ma, ep, K, n_tiles, m_tiles);
  return launched(1);
}

// CTA pairs resident at a time for a pair kernel (clusters of 2 with its shared memory), cached per device.
template <class Kernel>
int max_active_pairs(Kernel kernel, int smem, PerDevice& cache) {
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = cache.v[dev].load(std::memory_order_acquire);
  if (n > 0) return n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 0;
  }
  cache.v[dev].store(n, std::memory_order_release);
  return n;
}

template <int TA>
int launch_exact_pair(const CUtensorMap& mw, const CUtensorMap& mb, const ExactEpiParams& ep, int K, cudaStream_t st) {
  using Cfg = PairCfg<3, 3, TA>;
  static PerDevice configured, pairs_cache;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_pair_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int pairs = max_active_pairs(exact_linear_pair_kernel<TA>, Cfg::SMEM_BYTES, pairs_cache);
  if (pairs <= 0) return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles2 = (ep.N + 2 * WROWS - 1) / (2 * WROWS);
  const int total = m_tiles * n_tiles2;
  const int grid = 2 * (total < pairs ? total : pairs);
  exact_linear_pair_kernel<TA><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mw, mb, ep, K, n_tiles2, m_tiles);
  return launched(1);
}

template <int TN, bool DBL>
int launch_exact_rows(const CUtensorMap& ma, const CUtensorMap& mw, const ExactEpiParams& ep, int K, cudaStream_t st) {
  using Cfg = RowsCfg<TN, DBL>;
  static PerDevice configured, pairs_cache;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_rows_kernel<TN, DBL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int pairs = max_active_pairs(exact_linear_rows_kernel<TN, DBL>, Cfg::SMEM_BYTES, pairs_cache);
  if (pairs <= 0) return BX_ELAUNCH;
  const int n_tiles = (ep.N + TN - 1) / TN;
  const int m_tiles2 = (ep.M + 2 * WROWS - 1) / (2 * WROWS);
  const long total = (long)n_tiles * m_tiles2;
  const int grid = 2 * (int)(total < pairs ? total : pairs);
  exact_linear_rows_kernel<TN, DBL><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(ma, mw, ep, K, n_tiles, m_tiles2);
  return launched(1);
}

template <int TN, int NBUF>
int launch_exact_rows_one(const CUtensorMap& mact, const CUtensorMap& mwt, const ExactEpiParams& ep, int K,
                          cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TN>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(exact_linear_rows_one_kernel<TN, NBUF>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int sms = device_sms();
  if (sms <= 0) return BX_ELAUNCH;
  const int row_blocks = (ep.M + WROWS - 1) / WROWS;
  const int w_tiles = (ep.N + TN - 1) / TN;
  const long total = (long)row_blocks * w_tiles;
  const int grid = (int)(total < sms ? total : sms);
  exact_linear_rows_one_kernel<TN, NBUF><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mact, mwt, ep, K, row_blocks,
                                                                                     w_tiles);
  return launched(1);
}

template <int TA, bool POST>
int launch_int8(const CUtensorMap& mw, const CUtensorMap& ma, const Int8EpiParams& ep, int K, cudaStream_t st) {
  using Cfg = GemmCfg<1, 2, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(int8_linear_kernel<TA, POST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  int8_linear_kernel<TA, POST><<<m_tiles * n_tiles, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mw, ma, ep, K, m_tiles);
  return launched(1);
}

template <int TA, bool POST>
int launch_int8_persistent(const CUtensorMap& mw, const CUtensorMap& ma, const Int8EpiParams& ep, int K,
                           cudaStream_t st) {
  using Cfg = GemmCfg<1, 2, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(int8_linear_persistent_kernel<TA, POST>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int sms = device_sms();
  if (sms <= 0) return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  const int total = m_tiles * n_tiles;
  const int grid = total < sms ? total : sms;
  int8_linear_persistent_kernel<TA, POST><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mw, ma, ep, K, n_tiles, m_tiles);
  return launched(1);
}

template <int TA>
int launch_int8_splitk(const CUtensorMap& mw, const CUtensorMap& ma, const Int8EpiParams& ep, int K, int split,
                       cudaStream_t st) {
  using Cfg = GemmCfg<1, 2, TA>;
  static_assert((TA + SPLITK_MAX - 1) * WROWS * 8 <= Cfg::STAGES * Cfg::STAGE_BYTES, "partial columns fit in the ring");
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(int8_linear_splitk_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(m_tiles * n_tiles * split), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, int8_linear_splitk_kernel<TA>, mw, ma, ep, K, m_tiles) != cudaSuccess) return BX_ELAUNCH;
  return launched(1);
}

template <int TA>
int launch_bmm_limb(const CUtensorMap& mb, const CUtensorMap& ma, const BmmEpiParams& ep, int Z, int K16, cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TA>;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(bmm_limb_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int m_tiles = (ep.M + TA - 1) / TA, n_tiles = (ep.N + WROWS - 1) / WROWS;
  const long grid = (long)Z * m_tiles * n_tiles;
  if (grid > 0x7fffffffL) return BX_EARG;
  bmm_limb_kernel<TA><<<(unsigned)grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mb, ma, ep, K16, n_tiles, m_tiles);
  return launched(1);
}

template <class TX>
void launch_bmm_pack(const void* x, int64_t sz, int64_t sr, int64_t sk, int8_t* planes, int Z, int R, int K, int K16,
                     cudaStream_t st) {
  const int64_t total = (int64_t)Z * R * (K16 / 16);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  bmm_pack_kernel<TX><<<(unsigned)blocks, 256, 0, st>>>((const TX*)x, sz, sr, sk, planes, Z, R, K, K16);
}

template <bool POST>
int run_int8(const int8_t* a, const int8_t* w, const Int8EpiParams& ep, int K, int tile_rows, cudaStream_t st) {
  const int M = ep.M, N = ep.N;
  if (!a || !w || M < 0 || N <= 0 || K <= 0 || K % 16 || K >= 65536 || !aligned16(a) || !aligned16(w)) return BX_EARG;
  if (M == 0) return BX_OK;
  int ta = tile_rows;
  bool persistent = false;
  if (ta < 0) {                       // negative: that tile size on the persistent kernel
    ta = -ta;
    persistent = true;
  } else if (ta == 0) {
    const long n_tiles = (N + WROWS - 1) / WROWS;
    ta = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : (n_tiles * ((M + 127) / 128) >= 90 ? 128 : 64);
    // 64-row tiles that would cover less than half of the SMs: with a short K, 32-row tiles (wo at 256 rows:
    // 12.7 -> 10.6 us); with a long K the 64-row tiles stay and K is split over clusters below
    if (ta == 64 && M > 64 && K < 4096 && n_tiles * ((M + 63) / 64) * 2 <= 148) ta = 32;
    // more tiles than SMs: one CTA per SM with the epilogue of a tile behind the MMAs of the next
    persistent = n_tiles * ((M + ta - 1) / ta) > 148;
  }
  // Split-K over a cluster of CTAs (fused post only): 200 + rows (10000 S + 200 + rows: clusters of exactly S) asks
  // for it; automatic when the tile list covers less than half of the SMs and K is long enough for two K blocks per
  // slice, with as many slices (2, 4 or 8) as keep the CTA count within the SMs.
  int split = 0;
  if (POST) {
    int want = 0;
    if (ta >= 10000) { want = ta / 10000; ta %= 10000; if (want != 2 && want != 4 && want != 8) return BX_EARG; }
    if (ta >= 200 && ta < 300) {
      ta -= 200;
      if (ta != 16 && ta != 32 && ta != 64) return BX_EARG;
      split = want ? want : SPLITK_MAX;
    } else if (want) {
      return BX_EARG;
    } else if (tile_rows == 0 && !persistent && (ta == 16 || ta == 32 || ta == 64)) {
      const long tiles = ((N + WROWS - 1) / WROWS) * (long)((M + ta - 1) / ta);
      if (tiles * 2 <= 148) split = (int)(148 / tiles);
      if (split > 8) split = 8;
    }
    if (split > 0) {
      const int nkb = (K + BKB - 1) / BKB;
      if (split > nkb / 2) split = nkb / 2;
      while (split & (split - 1)) --split;
      if (tile_rows == 0 && split > 4) split = 4;
    }
  }
  CUtensorMap mw, ma;
  if (!make_map(&mw, w, (uint64_t)K, (uint64_t)N, 1, WROWS)) return BX_ELAUNCH;
  if (!make_map(&ma, a, (uint64_t)K, (uint64_t)M, 2, (uint32_t)ta)) return BX_ELAUNCH;
  if constexpr (POST) {
    if (split >= 2) {
      switch (ta) {
        case 16: return launch_int8_splitk<16>(mw, ma, ep, K, split, st);
        case 32: return launch_int8_splitk<32>(mw, ma, ep, K, split, st);
        default: return launch_int8_splitk<64>(mw, ma, ep, K, split, st);
      }
    }
  }
  if (persistent) {
    switch (ta) {
      case 16: return launch_int8_persistent<16, POST>(mw, ma, ep, K, st);
      case 32: return launch_int8_persistent<32, POST>(mw, ma, ep, K, st);
      case 64: return launch_int8_persistent<64, POST>(mw, ma, ep, K, st);
      case 128: return launch_int8_persistent<128, POST>(mw, ma, ep, K, st);
      default: return BX_EARG;
    }
  }
  switch (ta) {
    case 16: return launch_int8<16, POST>(mw, ma, ep, K, st);
    case 32: return launch_int8<32, POST>(mw, ma, ep, K, st);
    case 64: return launch_int8<64, POST>(mw, ma, ep, K, st);
    case 128: return launch_int8<128, POST>(mw, ma, ep, K, st);
    default: return BX_EARG;
  }
}

}  // namespace

extern "C" {

int bx_version(void) { return 1; }

long long bx_launch_count(void) { return g_launches; }

int bx_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, bx::g_wait_timeouts, sizeof(int)) != cudaSuccess) return BX_ELAUNCH;
  if (v != 0) g_status_seen.store(1);
  return v;
}

int bx_clear_device_status(void) {
  int v = 0;
  if (cudaMemcpyToSymbol(bx::g_wait_timeouts, &v, sizeof(int)) != cudaSuccess) return BX_ELAUNCH;
  g_status_seen.store(0);
  return BX_OK;
}

int bx_set_device_status(int value) {
  if (value < 0) return BX_EARG;
  // Only the device word: the host-side shadow follows when the host next reads the word, exactly as after a
  // wait that really ran out on the device.
  if (cudaMemcpyToSymbol(bx::g_wait_timeouts, &value, sizeof(int)) != cudaSuccess) return BX_ELAUNCH;
  return BX_OK;
}

int bx_i8_tensor_peak(int iters, int repeats, double* tops, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (iters < 4 || iters > (1 << 22) || repeats < 1 || repeats > 64 || !tops) return BX_EARG;
  static PerDevice configured;
  if (once_per_device(configured, [] {
        return cudaFuncSetAttribute(i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PEAK_SMEM);
      }) != BX_OK)
    return BX_ELAUNCH;
  const int sms = device_sms();
  if (sms <= 0) return BX_ELAUNCH;
  cudaStream_t st = (cudaStream_t)stream;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess) return BX_ELAUNCH;
  if (cudaEventCreate(&e1) != cudaSuccess) { cudaEventDestroy(e0); return BX_ELAUNCH; }
  const double ops = (double)sms * iters * 4.0 * 2.0 * 128.0 * PEAK_N * 32.0;
  double best = 0.0, sum = 0.0;
  int rc = BX_OK;
  i8_peak_kernel<<<sms, 128, PEAK_SMEM, st>>>(iters / 4);          // warm-up
  for (int r = 0; r < repeats && rc == BX_OK; ++r) {
    cudaEventRecord(e0, st);
    i8_peak_kernel<<<sms, 128, PEAK_SMEM, st>>>(iters);
    cudaEventRecord(e1, st);
    float ms = 0.f;
    if (cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess || ms <= 0.f) {
      rc = BX_ELAUNCH;
      break;
    }
    const double t = ops / (ms * 1e-3) / 1e12;
    best = t > best ? t : best;
    sum += t;
    g_launches += 1;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc != BX_OK || cudaGetLastError() != cudaSuccess) return BX_ELAUNCH;
  tops[0] = best;
  tops[1] = sum / repeats;
  return BX_OK;
}

size_t bx_exact_linear_scratch_bytes(int M, int K) { return (size_t)3 * (size_t)M * (size_t)K; }

int bx_split_limbs(const int32_t* q, int64_t ldq, int8_t* a8, int M, int K, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!q || !a8 || M < 0 || K <= 0 || K % 16 || ldq % 4 || ldq < K || !aligned16(q) || !aligned16(a8)) return BX_EARG;
  if (M == 0) return BX_OK;
  const int64_t total = (int64_t)M * (K / 16);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  split_limbs_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, ldq, a8, M, K);
  return launched(1);
}

static int exact_linear_core(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                             const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                             const int8_t* planes, int64_t* y, int32_t* flag, int M, int N, int K, int checked,
                             int tile_rows, void* stream) {
  int8_t* scratch = const_cast<int8_t*>(planes);
  cudaStream_t st = (cudaStream_t)stream;
  int ta = tile_rows;
  bool persistent = false;
  if (ta < 0) {                       // negative: that tile size on the persistent kernel (16, 32, 48)
    ta = -ta;
    persistent = true;
    if (ta != 16 && ta != 32 && ta != 48) return BX_EARG;
  } else if (ta == 0) {
    // Activation rows per CTA: the size that needs the fewest wave-rows (below); a tile list of more than two waves
    // goes to the persistent kernel (48 rows, overlapped epilogue).
    const long n_tiles = (N + WROWS - 1) / WROWS;
    ta = M <= 16 ? 16 : M <= 32 ? 32 : 48;
    if (M > 48) {
      // waves of 148 CTAs x (rows of a tile + a fixed cost of about 16 rows' worth of prologue and epilogue)
      long best = -1;
      const int cand[3] = {64, 48, 32};
      for (int i = 0; i < 3; ++i) {
        const long tiles = n_tiles * ((M + cand[i] - 1) / cand[i]);
        const long cost = ((tiles + 147) / 148) * (cand[i] + 16);
        if (best < 0 || cost < best) { best = cost; ta = cand[i]; }
      }
    }
    if (ta <= 48 && n_tiles * ((M + ta - 1) / ta) > 2 * 148) persistent = true;
    if (ta == 64 && K <= 4096 && n_tiles * ((M + 47) / 48) > 2 * 148) { ta = 48; persistent = true; }
    // Long tile lists of batches that fill blocks of 128 rows about as well as tiles of 48: the activation rows go
    // to the MMA M side, 64 weight rows per tile (no ragged sixth tile at 256 rows, warp-uniform residual lists,
    // wider MMAs). Measured, gate / up and LM head: 80 -> 67 us and 519 -> 429 us at M = 256, 46 -> 42 us and
    // 277 -> 238 us at M = 128, gate / up 878 -> 809 us at M = 4096.
    if (persistent && ta == 48 && M >= WROWS) {
      const long ra = ((M + WROWS - 1) / WROWS) * (long)WROWS, rw = ((M + 47) / 48) * 48L;
      if (10 * ra <= 11 * rw) ta = 664;
    }
  }
  int want_split = 0;                 // 10000 S + 200 + rows: split-K over clusters of exactly S CTAs
  if (ta >= 10000) {
    want_split = ta / 10000;
    ta %= 10000;
    if (!((ta >= 200 && ta < 300) || ta == 764) || (want_split != 2 && want_split != 4 && want_split != 8)) return BX_EARG;
  }
  // Long K, few tiles, a batch that fills blocks of 128 rows (the down projection at 256 rows): K split over CTA
  // pairs with the activation rows on the MMA M side, 64 weight rows per tile (764; 10000 S + 764: clusters of S).
  if (tile_rows == 0 && !persistent && M >= WROWS && K >= 8192 &&
      10 * (((M + WROWS - 1) / WROWS) * (long)WROWS) <= 11 * (((M + 47) / 48) * 48L) &&
      ((M + WROWS - 1) / WROWS) * (long)((N + 63) / 64) * 2 <= 148) {
    const long tiles = ((M + WROWS - 1) / WROWS) * (long)((N + 63) / 64);
    ta = 764;
    want_split = tiles * 4 <= 148 ? 4 : 2;           // as many K slices as keep the CTA count within the SMs
  }
  if (ta == 764) {
    int split = want_split ? want_split : 2;
    const int nkb = (K + BKB - 1) / BKB;
    if (split > nkb / 2) split = nkb / 2;
    while (split & (split - 1)) --split;
    if (split >= 2) {
      CUtensorMap mact, mwt;
      if (!make_map(&mact, scratch, (uint64_t)K, (uint64_t)M, 3, WROWS)) return BX_ELAUNCH;
      if (!make_map(&mwt, limbs, (uint64_t)K, (uint64_t)N, 3, 64)) return BX_ELAUNCH;
      ExactEpiParams ep{q, ldq, sh, d, g, cnt, ec, ev, R, y, flag, M, N, checked};
      return launch_exact_rows_splitk<64>(mact, mwt, ep, K, split, st);
    }
    ta = 664;                          // K too short to split: the same tile shape on the one-CTA kernel
  }
  // Split-K over a cluster of CTAs (200 + activation rows per tile asks for it; automatic for small batches whose
  // tile list covers less than half of the SMs): as many K slices as keep the CTA count within the 148 SMs.
  if (ta == 416 || ta == 432 || ta == 448) {          // 400 + rows: that tile size on the CTA-pair kernel
    ta -= 400;
    CUtensorMap mw, mb;
    if (!make_map(&mw, limbs, (uint64_t)K, (uint64_t)N, 3, WROWS)) return BX_ELAUNCH;
    if (!make_map_chunks(&mb, scratch, (uint64_t)K, (uint64_t)M, 3, (uint32_t)(ta / 2))) return BX_ELAUNCH;
    ExactEpiParams ep{q, ldq, sh, d, g, cnt, ec, ev, R, y, flag, M, N, checked};
    switch (ta) {
      case 16: return launch_exact_pair<16>(mw, mb, ep, K, st);
      case 32: return launch_exact_pair<32>(mw, mb, ep, K, st);
      default: return launch_exact_pair<48>(mw, mb, ep, K, st);
    }
  }
  if (ta == 516 || ta == 532 || ta == 548 || ta == 564 || ta == 580) {
    // 500 + weight rows per tile: activation rows on the MMA M side, CTA pairs (16 .. 48: two accumulator buffers)
    ta -= 500;
    CUtensorMap ma, mw;
    if (!make_map(&ma, scratch, (uint64_t)K, (uint64_t)M, 3, WROWS)) return BX_ELAUNCH;
    if (!make_map_chunks(&mw, limbs, (uint64_t)K, (uint64_t)N, 3, (uint32_t)(ta / 2))) return BX_ELAUNCH;
    ExactEpiParams ep{q, ldq, sh, d, g, cnt, ec, ev, R, y, flag, M, N, checked};
    switch (ta) {
      case 16: return launch_exact_rows<16, true>(ma, mw, ep, K, st);
      case 32: return launch_exact_rows<32, true>(ma, mw, ep, K, st);
      case 48: return launch_exact_rows<48, true>(ma, mw, ep, K, st);
      case 64: return launch_exact_rows<64, false>(ma, mw, ep, K, st);
      default: return launch_exact_rows<80, false>(ma, mw, ep, K, st);
    }
  }
  if (ta == 616 || ta == 632 || ta == 648 || ta == 664 || ta == 680) {
    // 600 + weight rows per tile: activation rows on the MMA M side, one CTA (16 .. 48: two accumulator buffers)
    ta -= 600;
    CUtensorMap mact, mwt;
    if (!make_map(&mact, scratch, (uint64_t)K, (uint64_t)M, 3, WROWS)) return BX_ELAUNCH;
    if (!make_map(&mwt, limbs, (uint64_t)K, (uint64_t)N, 3, (uint32_t)ta)) return BX_ELAUNCH;
    ExactEpiParams ep{q, ldq, sh, d, g, cnt, ec, ev, R, y, flag, M, N, checked};
    switch (ta) {
      case 16: return launch_exact_rows_one<16, 2>(mact, mwt, ep, K, st);
      case 32: return launch_exact_rows_one<32, 2>(mact, mwt, ep, K, st);
      case 48: return launch_exact_rows_one<48, 2>(mact, mwt, ep, K, st);
      case 64: return launch_exact_rows_one<64, 1>(mact, mwt, ep, K, st);
      default: return launch_exact_rows_one<80, 1>(mact, mwt, ep, K, st);
    }
  }
  int split = 0;
  if (ta >= 200) {
    ta -= 200;
    split = want_split ? want_split : SPLITK_MAX;
    if (ta != 16 && ta != 32 && ta != 64) return BX_EARG;
  } else if (tile_rows == 0 && !persistent && M <= 128 && (ta == 16 || ta == 32 || ta == 64)) {
    const long tiles = ((N + WROWS - 1) / WROWS) * ((M + ta - 1) / ta);
    if (tiles * 2 <= 148) split = (int)(148 / tiles);
  } else if (tile_rows == 0 && !persistent && M > 128 && K >= 8192 &&
             ((N + WROWS - 1) / WROWS) * (long)((M + 63) / 64) * 2 <= 148) {
    // Long K, few tiles (the down projection at a batch of 256): 64-row tiles with K split over CTA pairs read less
    // shared memory per product than one wave of 32-row tiles (measured 47 -> 39 us).
    ta = 64;
    split = 2;
  }
  if (split > 0) {
    const int nkb = (K + BKB - 1) / BKB;
    const int lim = ta == 16 ? splitk_limit<16>() : ta == 32 ? splitk_limit<32>() : splitk_limit<64>();
    if (split > lim) split = lim;
    if (split > nkb / 2) split = nkb / 2;                      // at least two K blocks per slice
    while (split & (split - 1)) --split;   // clusters of 2, 4 or 8: a cluster of 6 ran 1.6 x slower than one of 4
    // automatic choice: at most 4 (clusters of 8 measured 1.3 - 1.5 x slower on these shapes: fewer of them are
    // resident at a time); an explicit request (tile_rows 2xx) may still take 8
    if (tile_rows == 0 && split > 4) split = 4;
  }
  CUtensorMap mw, ma;
  if (!make_map(&mw, limbs, (uint64_t)K, (uint64_t)N, 3, WROWS)) return BX_ELAUNCH;
  if (!make_map(&ma, scratch, (uint64_t)K, (uint64_t)M, 3, (uint32_t)ta)) return BX_ELAUNCH;
  ExactEpiParams ep{q, ldq, sh, d, g, cnt, ec, ev, R, y, flag, M, N, checked};
  if (split >= 2) {
    switch (ta) {
      case 16: return launch_exact_splitk<16>(mw, ma, ep, K, split, st);
      case 32: return launch_exact_splitk<32>(mw, ma, ep, K, split, st);
      default: return launch_exact_splitk<64>(mw, ma, ep, K, split, st);
    }
  }
  if (persistent) {
    switch (ta) {
      case 16: return launch_exact_persistent<16>(mw, ma, ep, K, st);
      case 32: return launch_exact_persistent<32>(mw, ma, ep, K, st);
      default: return launch_exact_persistent<48>(mw, ma, ep, K, st);
    }
  }
  switch (ta) {
    case 16: return launch_exact<16>(mw, ma, ep, K, st);
    case 32: return launch_exact<32>(mw, ma, ep, K, st);
    case 48: return launch_exact<48>(mw, ma, ep, K, st);
    case 64: return launch_exact<64>(mw, ma, ep, K, st);
    case 80: return launch_exact<80>(mw, ma, ep, K, st);
    default: return BX_EARG;
  }
}

int bx_exact_norm(int mode, const void* xin, const int64_t* yin, const int64_t* ids, const int64_t* gm,
                  const int64_t* ge, int64_t* xo, int32_t* q, int64_t* sh, int8_t* a8, int32_t* flag, int M, int D,
                  int do_norm, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!xin || !flag || M < 0 || D < 32 || D > 4096 || (D & (D - 1))) return BX_EARG;
  if ((mode == 0 && !ids) || (mode == 1 && !yin) || mode < 0 || mode > 2) return BX_EARG;
  if (do_norm && (!gm || !ge || !q || !sh)) return BX_EARG;
  if (M == 0) return BX_OK;
  int lg = 0;
  while ((1 << lg) < D) ++lg;
  cudaStream_t st = (cudaStream_t)stream;
  const i64* y = (const i64*)yin; const i64* id = (const i64*)ids;
#define BX_NORM_LAUNCH(MODE, NT, EPT) \
  norm_kernel<MODE, NT, EPT><<<M, NT, 0, st>>>(xin, y, id, (const i64*)gm, (const i64*)ge, (i64*)xo, q, (i64*)sh, a8, \
                                              flag, M, D, lg, do_norm)
  if (D <= 2048) {                      // 512 threads x 4 elements
    if (mode == 0) BX_NORM_LAUNCH(0, 512, 4); else if (mode == 1) BX_NORM_LAUNCH(1, 512, 4); else BX_NORM_LAUNCH(2, 512, 4);
  } else {                              // 512 threads x 8 elements
    if (mode == 0) BX_NORM_LAUNCH(0, 512, 8); else if (mode == 1) BX_NORM_LAUNCH(1, 512, 8); else BX_NORM_LAUNCH(2, 512, 8);
  }
#undef BX_NORM_LAUNCH
  return launched(1);
}

int bx_exact_qkv(const int64_t* y, const int64_t* cos, const int64_t* sin, const int64_t* pos,
                 const int64_t* slot, int8_t* cache, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, int32_t* q,
                 int64_t* sh, int32_t* flag, int N, int H, int HKV, int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !cos || !sin || !pos || !q || !sh || !flag || N < 0) return BX_EARG;
  if ((HD != 64 && HD != 128) || HKV <= 0 || H % HKV || (cache && (!slot || bs <= 0))) return BX_EARG;
  if (N == 0) return BX_OK;
  QkvParams p{(const i64*)y, (const i64*)cos, (const i64*)sin, (const i64*)pos, (const i64*)slot, cache, sc_nb, sc_h,
              sc_bs, bs, q, (i64*)sh, flag, H, HKV, HD};
  qkv_kernel<<<dim3(N, HKV), HD / 2, 0, (cudaStream_t)stream>>>(p);
  return launched(1);
}

int bx_kv_store(int8_t* cache, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const int64_t* slot,
                const int64_t* k, int64_t skz, int64_t skh, const int64_t* v, int64_t svz, int64_t svh, int N,
                int HKV, int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!cache || !slot || !k || !v || bs <= 0 || N < 0 || HKV <= 0 || HD <= 0) return BX_EARG;
  if (N == 0) return BX_OK;
  kv_store_kernel<<<dim3(N, HKV), 64, 0, (cudaStream_t)stream>>>(cache, (const i64*)slot, (const i64*)k, (const i64*)v,
                                                                 skz, skh, svz, svh, sc_nb, sc_h, sc_bs, bs, HD);
  return launched(1);
}

int bx_exact_attn_out(const int64_t* num, const int64_t* den, int32_t* q, int64_t* sh, int8_t* a8, int N, int K2,
                      int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!num || !den || !q || !sh || N < 0 || K2 <= 0 || K2 > AO_THREADS * AO_EPT || HD <= 0 || K2 % HD ||
      K2 / HD > AO_MAXH)
    return BX_EARG;
  if (N == 0) return BX_OK;
  attn_out_kernel<<<N, AO_THREADS, 0, (cudaStream_t)stream>>>((const i64*)num, (const i64*)den, q, (i64*)sh, a8, N, K2, HD);
  return launched(1);
}

int bx_exact_silu_quant(const int64_t* y, const int64_t* lut, int32_t* q, int64_t* sh, int8_t* a8, int32_t* flag,
                        int N, int FF, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !lut || !q || !sh || !flag || N < 0 || FF <= 0 || FF > SILU_THREADS * 28) return BX_EARG;
  if (N == 0) return BX_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (FF <= 8 * SILU_P_THREADS && N >= 64) {        // one persistent CTA per SM, 2^-f table in shared memory
    static PerDevice configured;
    const int smem = SILU_TABLE * 8;
    if (once_per_device(configured, [smem] {
          return cudaFuncSetAttribute(silu_persistent_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        }) != BX_OK)
      return BX_ELAUNCH;
    const int sms = device_sms();
    if (sms <= 0) return BX_ELAUNCH;
    // equal rounds: with 256 rows, 128 CTAs of two rows each rather than 148 CTAs of one or two
    const int rounds = (N + sms - 1) / sms;
    const int grid = (N + rounds - 1) / rounds;
    silu_persistent_kernel<8><<<grid, SILU_P_THREADS, smem, st>>>((const i64*)y, (const i64*)lut, q, (i64*)sh, a8, flag,
                                                                  N, FF);
    return launched(1);
  }
  if (FF == SILU_CL * SILU_CL_THREADS * 8 && N <= 4096) {          // decode batches of the 1B model: cluster form
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SILU_CL * N, 1, 1);
    cfg.blockDim = dim3(SILU_CL_THREADS, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SILU_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, silu_cluster_kernel<8>, (const i64*)y, (const i64*)lut, q, (i64*)sh, a8, flag, N, FF) !=
        cudaSuccess)
      return BX_ELAUNCH;
    return launched(1);
  }
  const int ept = (FF + SILU_THREADS - 1) / SILU_THREADS;
  if (ept <= 4) silu_kernel<4><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, q, (i64*)sh, a8, flag, N, FF);
  else if (ept <= 16) silu_kernel<16><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, q, (i64*)sh, a8, flag, N, FF);
  else silu_kernel<28><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, q, (i64*)sh, a8, flag, N, FF);
  return launched(1);
}

// Persistent streaming kernel (variants 5: 8 consumer warps, 6: 4 consumer warps). BX_ENOFIT: too few pairs or a
// context whose scores do not fit beside the ring (the caller falls back to the cluster kernels unless the variant
// was asked for explicitly).
constexpr int BX_ENOFIT = -100;

static int run_attention_stream(int NW, const int32_t* q, const int64_t* sh, const int64_t* qpos, const int8_t* cache,
                                int64_t nb, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const void* bt,
                                int bt_is_int64, int64_t sbt, int nblk, const int64_t* rmap, const int64_t* lut,
                                int64_t l2e, const int32_t* ptab, int64_t* num, int64_t* den, int R, int HKV, int M,
                                int min_per_sm, void* spill, size_t spill_bytes, void* stream) {
  const bool forced = min_per_sm == 0;                          // an explicit variant: any fit will do
  const int KEYS = 8 * NW, STAGE = KEYS * 256;
  const int64_t max_keys = (int64_t)nblk * bs;
  const int64_t npairs = (int64_t)R * HKV;
  if (bs > KEYS || KEYS % bs != 0 || 32 % bs != 0) return forced ? BX_EARG : BX_ENOFIT;
  if (!forced && npairs < 2 * 148) return BX_ENOFIT;
  // Scores in shared memory for the whole context, or (scratch given) chunks of 512 keys with the scores of longer
  // pairs in the caller's scratch buffer, one slice per CTA.
  const int64_t spill_keys = (max_keys + 63) / 64 * 64;
  const bool chunked = spill != nullptr;
#ifndef BX_ATT_CHUNK
#define BX_ATT_CHUNK 512
#endif
  const int64_t cap = chunked ? BX_ATT_CHUNK : (max_keys + KEYS - 1) / KEYS * KEYS;     // chunks: a multiple of 32 NW keys
  if (cap / 32 > ATT6_MAXGROUPS) return forced ? BX_EARG : BX_ENOFIT;
  const int64_t fixed = 1024 + cap * 32 + (int64_t)sizeof(Attn6Small) + 1024 /* request order */;
  int per_sm = NW == 4 ? 4 : 2, ns = 0;
  for (; per_sm >= 1; --per_sm) {                               // most CTAs per SM that still leave a ring of 4 stages
    const int64_t budget = 227 * 1024 / per_sm - 1024;
    ns = (int)((budget - fixed) / STAGE);
    if (ns >= 4 || (per_sm == 1 && ns >= 3)) break;
  }
  if (per_sm < 1) return forced ? BX_EARG : BX_ENOFIT;
  if (!forced && per_sm < min_per_sm) return BX_ENOFIT;
  if (ns > ATT6_MAXNS) ns = ATT6_MAXNS;
  const size_t smem = (size_t)fixed + (size_t)ns * STAGE;
  AttnParams p{q, (const i64*)sh, (const i64*)qpos, cache, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk,
               (const i64*)rmap, (const i64*)lut, (i64)l2e, (i64*)num, (i64*)den, M, HKV, (int)cap, ptab};
  static PerDevice configured;
  if (once_per_device(configured, [] {
        cudaError_t e = cudaFuncSetAttribute(exact_attention_stream_kernel<8>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        return e != cudaSuccess ? e
                                : cudaFuncSetAttribute(exact_attention_stream_kernel<4>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      }) != BX_OK)
    return BX_ELAUNCH;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return BX_ELAUNCH;
  CUtensorMap tk, tv;
  cuuint64_t dims[4] = {512, (cuuint64_t)bs, (cuuint64_t)HKV, (cuuint64_t)nb};
  cuuint64_t strides[3] = {(cuuint64_t)sc_bs, (cuuint64_t)sc_h, (cuuint64_t)sc_nb};
  cuuint32_t boxk[4] = {ATT2_HALF, (cuuint32_t)bs, 1, 1};
  cuuint32_t boxv[4] = {128, (cuuint32_t)bs, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  // 64-byte L2 promotion on both maps: measured against none / 128 B / 256 B, it is the only setting that changes
  // anything (batch 256, contexts U[64, 8192]: 875 -> 817 us; neutral at short contexts; 256 B: 15 % slower).
  if (fn(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(cache), dims, strides, boxk, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_64B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
      fn(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(cache), dims, strides, boxv, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_64B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return BX_ELAUNCH;
  const int64_t grid = npairs < (int64_t)per_sm * 148 ? npairs : (int64_t)per_sm * 148;
  if (chunked && (size_t)grid * (size_t)spill_keys * 32 > spill_bytes) return forced ? BX_EARG : BX_ENOFIT;
  if (NW == 8)
    exact_attention_stream_kernel<8><<<(unsigned)grid, 320, smem, (cudaStream_t)stream>>>(tk, tv, p, ns, npairs,
                                                                                          (i64*)spill, spill_keys);
  else
    exact_attention_stream_kernel<4><<<(unsigned)grid, 192, smem, (cudaStream_t)stream>>>(tk, tv, p, ns, npairs,
                                                                                          (i64*)spill, spill_keys);
  if (cudaGetLastError() != cudaSuccess) return BX_ELAUNCH;
  return launched(1);
}

static int run_attention(const int32_t* q, const int64_t* sh, const int64_t* qpos, const int8_t* cache, int64_t nb,
                         int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64,
                         int64_t sbt, int nblk, const int64_t* rmap, const int64_t* lut, int64_t l2e,
                         const int32_t* ptab, int64_t* num, int64_t* den, int R, int HKV, int M, int HD,
                         int cluster_size, int variant, void* spill, size_t spill_bytes, void* stream) {
  if (!q || !qpos || !cache || !bt || !num || !den) return BX_EARG;
  if (!ptab && (!sh || !lut)) return BX_EARG;
  if (R < 0 || HKV <= 0 || M < 1 || M > 4 || HD != ATT_HD || bs <= 0 || nblk <= 0 || nb <= 0) return BX_EARG;
  const int64_t max_keys = (int64_t)nblk * bs;
  if (max_keys >= 43690) return BX_EARG;
  if (R == 0) return BX_OK;
  const int64_t smem_limit = 227 * 1024;
  // TMA-staged kernel when the cache layout allows a tensor map over it, else the direct-load kernel.
  const bool tma_ok = (bs % 8 == 0) && (ATT2_STAGE_KEYS % bs == 0) && sc_bs % 16 == 0 && sc_h % 16 == 0 &&
                      sc_nb % 16 == 0 && sc_bs >= 384 && aligned16(cache);
  if (variant >= 2 && !tma_ok) return BX_EARG;
  if (variant < 0 || variant > 6 || (variant == 4 && bs > 32)) return BX_EARG;
  // 5 / 6: persistent streaming kernel (8 / 4 consumer warps). Automatic choice, by CTAs that fit on an SM beside the
  // score buffer: four 4-warp CTAs, else two 8-warp CTAs, else two or three 4-warp CTAs; with a single CTA per SM
  // the cluster kernels below stream better.
  if (variant == 0 && tma_ok) {
    const int tries[3][2] = {{4, 4}, {8, 2}, {4, 2}};
    for (int t = 0; t < 3; ++t) {
      const int rc = run_attention_stream(tries[t][0], q, sh, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64,
                                          sbt, nblk, rmap, lut, l2e, ptab, num, den, R, HKV, M, tries[t][1], nullptr, 0,
                                          stream);
      if (rc != BX_ENOFIT) return rc;
    }
    if (spill) {                                                // long contexts: chunks of 512 keys, scores in scratch
      const int rc = run_attention_stream(4, q, sh, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk,
                                          rmap, lut, l2e, ptab, num, den, R, HKV, M, 3, spill, spill_bytes, stream);
      if (rc != BX_ENOFIT) return rc;
    }
  }
  if (variant == 5 || variant == 6)
    return run_attention_stream(variant == 5 ? 8 : 4, q, sh, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64,
                                sbt, nblk, rmap, lut, l2e, ptab, num, den, R, HKV, M, 0, spill, spill_bytes, stream);
  // 1 direct loads, 2 TMA-staged, 3 TMA + tcgen05 p.V with 8 consumer warps, 4 the same with 4 consumer warps
  const int kind = variant != 0 ? variant : (tma_ok ? ((bs <= 32 && (int64_t)R * HKV >= 64) ? 4 : 3) : 1);
  const int nw = kind == 4 ? 4 : 8;
  const bool use_tma = kind >= 2;
  const int64_t fixed = kind >= 3 ? 1024 + (int64_t)ATT3_NS * (8 * nw * 256) + (int64_t)sizeof(Attn3Small)
                        : kind == 2 ? (int64_t)ATT2_NS * ATT2_STAGE_BYTES + (int64_t)sizeof(Attn2Small)
                                    : (int64_t)sizeof(AttnShared);
  const int64_t gran = kind >= 3 ? 8 * nw : use_tma ? ATT2_STAGE_KEYS : 8;
  const int64_t cap_limit = (smem_limit - fixed) / 32 / gran * gran;
  int cs = cluster_size;
  if (cs == 0) {
    cs = 1;
    const int64_t pairs = (int64_t)R * HKV;
    while (cs < ATT_MAXCS && pairs * cs < 2 * 148) cs *= 2;               // fill the SMs
    while (cs < ATT_MAXCS && (max_keys + cs - 1) / cs > (kind == 4 ? 512 : 704)) cs *= 2;   // small score buffer
  }
  if (cs != 1 && cs != 2 && cs != 4 && cs != 8) return BX_EARG;
  auto cap_of = [&](int c) { return ((max_keys + c - 1) / c + gran - 1) / gran * gran; };
  while (cs < ATT_MAXCS && cap_of(cs) > cap_limit) cs *= 2;
  const int chunk_cap = (int)cap_of(cs);
  if (chunk_cap > cap_limit) return BX_EARG;
  const size_t smem = (size_t)fixed + (size_t)chunk_cap * 32;
  AttnParams p{q, (const i64*)sh, (const i64*)qpos, cache, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk,
               (const i64*)rmap, (const i64*)lut, (i64)l2e, (i64*)num, (i64*)den, M, HKV, chunk_cap, ptab};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((int64_t)cs * R * HKV), 1, 1);
  cfg.blockDim = dim3(kind == 4 ? 160 : use_tma ? ATT2_THREADS : ATT_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  static PerDevice configured[5];
  if (once_per_device(configured[kind], [kind, smem_limit] {
        return kind == 4 ? cudaFuncSetAttribute(exact_attention_tc_kernel<4>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit)
               : kind == 3 ? cudaFuncSetAttribute(exact_attention_tc_kernel<8>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit)
               : kind == 2 ? cudaFuncSetAttribute(exact_attention_tma_kernel,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit)
                           : cudaFuncSetAttribute(exact_attention_kernel,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit);
      }) != BX_OK)
    return BX_ELAUNCH;
  if (kind >= 3) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return BX_ELAUNCH;
    CUtensorMap tk, tv;
    cuuint64_t dims[4] = {512, (cuuint64_t)bs, (cuuint64_t)HKV, (cuuint64_t)nb};
    cuuint64_t strides[3] = {(cuuint64_t)sc_bs, (cuuint64_t)sc_h, (cuuint64_t)sc_nb};
    cuuint32_t boxk[4] = {ATT2_HALF, (cuuint32_t)bs, 1, 1};
    cuuint32_t boxv[4] = {128, (cuuint32_t)bs, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (fn(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(cache), dims, strides, boxk, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
        fn(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(cache), dims, strides, boxv, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return BX_ELAUNCH;
    if ((kind == 4 ? cudaLaunchKernelEx(&cfg, exact_attention_tc_kernel<4>, tk, tv, p)
                   : cudaLaunchKernelEx(&cfg, exact_attention_tc_kernel<8>, tk, tv, p)) != cudaSuccess)
      return BX_ELAUNCH;
  } else if (use_tma) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return BX_ELAUNCH;
    CUtensorMap tm;
    cuuint64_t dims[4] = {512, (cuuint64_t)bs, (cuuint64_t)HKV, (cuuint64_t)nb};
    cuuint64_t strides[3] = {(cuuint64_t)sc_bs, (cuuint64_t)sc_h, (cuuint64_t)sc_nb};
    cuuint32_t box[4] = {ATT2_HALF, (cuuint32_t)bs, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (fn(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(cache), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return BX_ELAUNCH;
    if (cudaLaunchKernelEx(&cfg, exact_attention_tma_kernel, tm, p) != cudaSuccess) return BX_ELAUNCH;
  } else {
    if (cudaLaunchKernelEx(&cfg, exact_attention_kernel, p) != cudaSuccess) return BX_ELAUNCH;
  }
  return launched(1);
}

int bx_exact_attention(const int32_t* q, const int64_t* sh, const int64_t* qpos, const int8_t* cache, int64_t nb,
                       int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64,
                       int64_t sbt, int nblk, const int64_t* rmap, const int64_t* lut, int64_t l2e, int64_t* num,
                       int64_t* den, int R, int HKV, int M, int HD, int cluster_size, int variant, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!sh || !lut) return BX_EARG;
  return run_attention(q, sh, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk, rmap, lut, l2e,
                       nullptr, num, den, R, HKV, M, HD, cluster_size, variant, nullptr, 0, stream);
}

size_t bx_attention_scratch_bytes(int nblk, int bs) {
  if (nblk <= 0 || bs <= 0) return 0;
  const size_t keys = ((size_t)nblk * bs + 63) / 64 * 64;
  return (size_t)4 * 148 * keys * 32;
}

int bx_exact_attention_ws(const int32_t* q, const int64_t* sh, const int64_t* qpos, const int8_t* cache, int64_t nb,
                          int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64,
                          int64_t sbt, int nblk, const int64_t* rmap, const int64_t* lut, int64_t l2e, int64_t* num,
                          int64_t* den, int R, int HKV, int M, int HD, int cluster_size, int variant, void* scratch,
                          size_t scratch_bytes, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!sh || !lut) return BX_EARG;
  return run_attention(q, sh, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk, rmap, lut, l2e,
                       nullptr, num, den, R, HKV, M, HD, cluster_size, variant, scratch, scratch_bytes, stream);
}

int bx_int8_attention_ws(const int32_t* q, const int64_t* qpos, const int8_t* cache, int64_t nb, int64_t sc_nb,
                         int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64, int64_t sbt, int nblk,
                         const int64_t* rmap, const int32_t* ptab, int64_t* num, int64_t* den, int R, int HKV, int M,
                         int HD, int cluster_size, int variant, void* scratch, size_t scratch_bytes, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!ptab) return BX_EARG;
  return run_attention(q, nullptr, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk, rmap, nullptr,
                       0, ptab, num, den, R, HKV, M, HD, cluster_size, variant, scratch, scratch_bytes, stream);
}

int bx_int8_attention(const int32_t* q, const int64_t* qpos, const int8_t* cache, int64_t nb, int64_t sc_nb,
                      int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64, int64_t sbt, int nblk,
                      const int64_t* rmap, const int32_t* ptab, int64_t* num, int64_t* den, int R, int HKV, int M,
                      int HD, int cluster_size, int variant, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!ptab) return BX_EARG;
  return run_attention(q, nullptr, qpos, cache, nb, sc_nb, sc_h, sc_bs, bs, bt, bt_is_int64, sbt, nblk, rmap, nullptr,
                       0, ptab, num, den, R, HKV, M, HD, cluster_size, variant, nullptr, 0, stream);
}

int bx_prefill_attention(const int32_t* q, const int64_t* sh, const int64_t* pos, const int32_t* tiles, int n_tiles,
                         const int8_t* cache, int64_t nb, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs,
                         const void* bt, int bt_is_int64, int64_t sbt, int nblk, const int64_t* lut, int64_t l2e,
                         const int32_t* ptab, int64_t* num, int64_t* den, int HKV, int G, int HD, int tile_rows,
                         void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!q || !pos || !tiles || !cache || !bt || !num || !den || n_tiles < 0) return BX_EARG;
  if (!ptab && (!sh || !lut)) return BX_EARG;
  if (tile_rows == 0) tile_rows = 32;
  if (tile_rows != 16 && tile_rows != 32) return BX_EARG;
  if (HD != ATT_HD || HKV <= 0 || HKV > 65535 || G < 1 || G > tile_rows || nblk <= 0 || nb <= 0) return BX_EARG;
  if (bs < 8 || bs > PF_KEYS || PF_KEYS % bs || (int64_t)nblk * bs >= 43690) return BX_EARG;
  if (sc_bs % 16 || sc_h % 16 || sc_nb % 16 || sc_bs < 384 || !aligned16(cache) || !aligned16(q)) return BX_EARG;
  if (n_tiles == 0) return BX_OK;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return BX_ELAUNCH;
  CUtensorMap tm;
  cuuint64_t dims[4] = {512, (cuuint64_t)bs, (cuuint64_t)HKV, (cuuint64_t)nb};
  cuuint64_t strides[3] = {(cuuint64_t)sc_bs, (cuuint64_t)sc_h, (cuuint64_t)sc_nb};
  cuuint32_t box[4] = {128, (cuuint32_t)bs, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (fn(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(cache), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return BX_ELAUNCH;
  const int smem32 = 2 * PF_STAGE + PfCfg<32>::QTILE + PfCfg<32>::PTILE + (int)sizeof(PrefillSmall) + 1024;
  const int smem16 = 2 * PF_STAGE + PfCfg<16>::QTILE + PfCfg<16>::PTILE + (int)sizeof(PrefillSmall) + 1024;
  static PerDevice configured;
  if (once_per_device(configured, [smem32, smem16] {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             smem32);
        return e != cudaSuccess ? e
                                : cudaFuncSetAttribute(prefill_attention_kernel<16>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem16);
      }) != BX_OK)
    return BX_ELAUNCH;
  PrefillParams p{};
  p.q = q;
  p.sh = (const i64*)sh;
  p.pos = (const i64*)pos;
  p.tiles = tiles;
  p.bt = bt;
  p.bt64 = bt_is_int64;
  p.sbt = sbt;
  p.nblk = nblk;
  p.bs = bs;
  p.w.lut = (const i64*)lut;
  p.w.l2e = (i64)l2e;
  p.w.ptab = ptab;
  p.num = (i64*)num;
  p.den = (i64*)den;
  p.HKV = HKV;
  p.G = G;
  const dim3 grid((unsigned)n_tiles, (unsigned)HKV);
  if (tile_rows == 32)
    prefill_attention_kernel<32><<<grid, PfCfg<32>::THREADS, smem32, (cudaStream_t)stream>>>(tm, p);
  else
    prefill_attention_kernel<16><<<grid, PfCfg<16>::THREADS, smem16, (cudaStream_t)stream>>>(tm, p);
  return launched(1);
}

int bx_int8_norm(int mode, const void* xin, const int64_t* yin, const int64_t* ids, const int64_t* gamma,
                 int64_t* xo, int8_t* a8, int64_t* mant, int64_t* e, int32_t* flag, int M, int D, int do_norm,
                 void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!xin || !flag || M < 0 || D < 1 || D > NORM_THREADS * NORM_EPT || mode < 0 || mode > 2) return BX_EARG;
  if ((mode == 0 && !ids) || (mode == 1 && !yin) || (do_norm && (!gamma || !a8 || !mant || !e))) return BX_EARG;
  if (M == 0) return BX_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == 0) i8::int8_norm_kernel<0><<<M, NORM_THREADS, 0, st>>>(xin, (const i64*)yin, (const i64*)ids, (const i64*)gamma, (i64*)xo, a8, (i64*)mant, (i64*)e, flag, M, D, do_norm);
  else if (mode == 1) i8::int8_norm_kernel<1><<<M, NORM_THREADS, 0, st>>>(xin, (const i64*)yin, (const i64*)ids, (const i64*)gamma, (i64*)xo, a8, (i64*)mant, (i64*)e, flag, M, D, do_norm);
  else i8::int8_norm_kernel<2><<<M, NORM_THREADS, 0, st>>>(xin, (const i64*)yin, (const i64*)ids, (const i64*)gamma, (i64*)xo, a8, (i64*)mant, (i64*)e, flag, M, D, do_norm);
  return launched(1);
}

int bx_int8_qkv(const int64_t* y, const int64_t* cos, const int64_t* sin, const int64_t* pos, const int64_t* slot,
                int8_t* cache, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, int64_t* q64, int32_t* q32,
                int32_t* flag, int N, int H, int HKV, int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !cos || !sin || !pos || !flag || (!q64 && !q32) || N < 0) return BX_EARG;
  if ((HD != 64 && HD != 128) || HKV <= 0 || H % HKV || (cache && (!slot || bs <= 0))) return BX_EARG;
  if (N == 0) return BX_OK;
  i8::Qkv8Params p{(const i64*)y, (const i64*)cos, (const i64*)sin, (const i64*)pos, (const i64*)slot, cache, sc_nb,
                   sc_h, sc_bs, bs, (i64*)q64, q32, flag, H, HKV, HD};
  i8::int8_qkv_kernel<<<dim3(N, HKV), HD / 2, 0, (cudaStream_t)stream>>>(p);
  return launched(1);
}

int bx_int8_attn_out(const int64_t* num, const int64_t* den, int8_t* a8, int64_t* mant, int64_t* e, int N, int K2,
                     int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!num || !den || !a8 || !mant || !e || N < 0 || K2 <= 0 || K2 > AO_THREADS * AO_EPT || HD <= 0 || K2 % HD ||
      K2 / HD > AO_MAXH)
    return BX_EARG;
  if (N == 0) return BX_OK;
  i8::int8_attn_out_kernel<<<N, AO_THREADS, 0, (cudaStream_t)stream>>>((const i64*)num, (const i64*)den, a8, (i64*)mant, (i64*)e, N, K2, HD);
  return launched(1);
}

int bx_int8_silu_quant(const int64_t* y, const int64_t* lut, int8_t* a8, int64_t* mant, int64_t* e, int64_t* scr,
                       int N, int FF, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !lut || !a8 || !mant || !e || N < 0 || FF <= 0 || FF > SILU_THREADS * 28) return BX_EARG;
  if (N == 0) return BX_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ept = (FF + SILU_THREADS - 1) / SILU_THREADS;
  if (ept <= 4) i8::int8_silu_kernel<4><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, a8, (i64*)mant, (i64*)e, (i64*)scr, N, FF);
  else if (ept <= 16) i8::int8_silu_kernel<16><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, a8, (i64*)mant, (i64*)e, (i64*)scr, N, FF);
  else i8::int8_silu_kernel<28><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, a8, (i64*)mant, (i64*)e, (i64*)scr, N, FF);
  return launched(1);
}

int bx_int8_silu_prod(const int64_t* y, const int64_t* lut, int64_t* h, int64_t* rowmax, int64_t* scr, int N, int FFl,
                      void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !lut || !h || !rowmax || N < 0 || FFl <= 0 || FFl > SILU_THREADS * 28) return BX_EARG;
  if (N == 0) return BX_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int ept = (FFl + SILU_THREADS - 1) / SILU_THREADS;
  if (ept <= 4) i8::int8_silu_prod_kernel<4><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, (i64*)h, (i64*)rowmax, (i64*)scr, N, FFl);
  else if (ept <= 16) i8::int8_silu_prod_kernel<16><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, (i64*)h, (i64*)rowmax, (i64*)scr, N, FFl);
  else i8::int8_silu_prod_kernel<28><<<N, SILU_THREADS, 0, st>>>((const i64*)y, (const i64*)lut, (i64*)h, (i64*)rowmax, (i64*)scr, N, FFl);
  return launched(1);
}

int bx_int8_quant_rows(const int64_t* h, const int64_t* rowmax, int8_t* a8, int64_t* mant, int64_t* e, int N, int K,
                       void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!h || !rowmax || !a8 || N < 0 || K <= 0 || (mant && !e)) return BX_EARG;
  if (N == 0) return BX_OK;
  i8::int8_quant_rows_kernel<<<N, 256, 0, (cudaStream_t)stream>>>((const i64*)h, (const i64*)rowmax, a8, (i64*)mant, (i64*)e, N, K);
  return launched(1);
}

int bx_int8_post(const int32_t* c, const int64_t* mul, int64_t fmsh, const int64_t* mant, const int64_t* e, int64_t* y,
                 int32_t* flag, int M, int N, int checked, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!c || !mul || !mant || !e || !y || !flag || M < 0 || N <= 0) return BX_EARG;
  if (M == 0) return BX_OK;
  const int64_t total = (int64_t)M * N;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  i8::int8_post_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(c, (const i64*)mul, (i64)fmsh, (const i64*)mant, (const i64*)e, (i64*)y, flag, M, N, checked);
  return launched(1);
}

int bx_int8_flag_end(int64_t* scr, int32_t* flag, int L, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!scr || !flag || L <= 0) return BX_EARG;
  i8::int8_flag_end_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((i64*)scr, flag, L);
  return launched(1);
}

int bx_pcg_raw(const int64_t* keys, int64_t* out, int n, int V, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!keys || !out || n < 0 || V <= 0) return BX_EARG;
  if (n == 0) return BX_OK;
  const int run = 16;
  const int blocks = (V + run * SAMPLE_THREADS - 1) / (run * SAMPLE_THREADS);
  pcg_raw_kernel<<<dim3(blocks, n), SAMPLE_THREADS, 0, (cudaStream_t)stream>>>((const i64*)keys, (i64*)out, V, run);
  return launched(1);
}

static int sample_chunks(int M, int V) {
  int nch = (8 * 148 + (M > 0 ? M : 1) - 1) / (M > 0 ? M : 1);       // eight 256-thread CTAs per SM
  const int maxch = (V + 2047) / 2048;
  if (nch > maxch) nch = maxch;
  return nch < 1 ? 1 : nch;
}

size_t bx_sample_scratch_bytes(int M, int V) { return (size_t)2 * 8 * (size_t)(M > 0 ? M : 0) * sample_chunks(M, V); }

static int run_sample(const int64_t* logits, int64_t ld, const int64_t* rows, const int64_t* lnt, void* scratch,
                      int64_t* tok, int64_t* omax, int M, int V, int64_t voff, int bits, void* stream) {
  if (!logits || !rows || !lnt || !scratch || !tok || M < 0 || V <= 0 || ld < V || voff < 0 || M > 65535) return BX_EARG;
  if (M == 0) return BX_OK;
  const int nch0 = sample_chunks(M, V);
  const int ch = ((V + nch0 - 1) / nch0 + 1) / 2 * 2;
  const int nch = (V + ch - 1) / ch;
  i64* pmax = (i64*)scratch;
  i64* pidx = pmax + (size_t)M * nch0;
  cudaStream_t st = (cudaStream_t)stream;
  sample_part_kernel<<<dim3(nch, M), SAMPLE_THREADS, 0, st>>>((const i64*)logits, ld, (const i64*)rows, (const i64*)lnt,
                                                              pmax, pidx, V, ch, nch, bits, (i64)voff);
  sample_combine_kernel<<<(M + 127) / 128, 128, 0, st>>>(pmax, pidx, (i64*)tok, (i64*)omax, M, nch);
  return launched(2);
}

int bx_sample(const int64_t* logits, int64_t ld, const int64_t* rows, const int64_t* lnt, void* scratch,
              int64_t* tok, int M, int V, int bits, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  return run_sample(logits, ld, rows, lnt, scratch, tok, nullptr, M, V, 0, bits, stream);
}

int bx_sample_shard(const int64_t* logits, int64_t ld, const int64_t* rows, const int64_t* lnt, void* scratch,
                    int64_t* best, int64_t* idx, int M, int V_local, int64_t v_offset, int bits, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!best) return BX_EARG;
  return run_sample(logits, ld, rows, lnt, scratch, idx, best, M, V_local, v_offset, bits, stream);
}

// ---- weight preparation (load time) ----
int bx_decompose_rows(const uint16_t* w, int64_t ldw, int8_t* limbs, int64_t* g, int64_t* d, int32_t* cnt, int32_t* flag,
                      int N, int K, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!w || !limbs || !g || !d || !cnt || !flag || N < 0 || K <= 0 || ldw < K) return BX_EARG;
  if (N == 0) return BX_OK;
  decompose_rows_kernel<<<N, DEC_THREADS, 0, (cudaStream_t)stream>>>(w, ldw, limbs, (i64*)g, (i64*)d, cnt, flag, N, K);
  return launched(1);
}

int bx_decompose_residual(const uint16_t* w, int64_t ldw, const int64_t* g, const int64_t* d, const int64_t* start,
                          int64_t* rr, int64_t* rc, int64_t* rv, int N, int K, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!w || !g || !d || !start || !rr || !rc || !rv || N < 0 || K <= 0 || ldw < K) return BX_EARG;
  if (N == 0) return BX_OK;
  decompose_residual_kernel<<<N, DEC_THREADS, 0, (cudaStream_t)stream>>>(w, ldw, (const i64*)g, (const i64*)d,
                                                                         (const i64*)start, (i64*)rr, (i64*)rc, (i64*)rv, K);
  return launched(1);
}

// ---- integer log p ----------------------------------------------------------------------------------------------
static void logp_plan(int M, int V, int& ch, int& nch) {
  const int nch0 = sample_chunks(M, V);
  ch = (V + nch0 - 1) / nch0;
  nch = (V + ch - 1) / ch;
}

size_t bx_logp_scratch_bytes(int M, int V) {
  return (size_t)2 * 8 * (size_t)(M > 0 ? M : 0) * sample_chunks(M, V > 0 ? V : 1);
}

static bool logp_args_ok(const void* lg, int64_t ld, const void* scratch, int M, int V) {
  return lg && scratch && M >= 0 && M <= 65535 && V > 0 && ld >= V;
}

int bx_logp_pair_table(const int64_t* tab, int tab_len, int64_t* tab2, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!tab || !tab2 || tab_len != LSE_LAST + 1 || ((uintptr_t)tab2 & 15)) return BX_EARG;
  logp_pair_table_kernel<<<(tab_len + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const i64*)tab, (longlong2*)tab2, tab_len);
  return launched(1);
}

int bx_logp_rowmax(const int64_t* logits, int64_t ld, void* scratch, int64_t* rowmax, int M, int V, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!logp_args_ok(logits, ld, scratch, M, V) || !rowmax) return BX_EARG;
  if (M == 0) return BX_OK;
  int ch, nch;
  logp_plan(M, V, ch, nch);
  cudaStream_t st = (cudaStream_t)stream;
  i64* pmax = (i64*)scratch;
  logp_max_kernel<<<dim3(nch, M), LOGP_THREADS, 0, st>>>((const i64*)logits, ld, pmax, V, ch, nch);
  logp_rowfold_kernel<<<(M + 127) / 128, 128, 0, st>>>(pmax, nch, (i64*)rowmax, M, 0);
  return launched(2);
}

int bx_logp_rowsum(const int64_t* logits, int64_t ld, const int64_t* rowmax, const int64_t* tab2, int tab_len,
                   void* scratch, int64_t* S, int M, int V, int fr, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!logp_args_ok(logits, ld, scratch, M, V) || !rowmax || !tab2 || ((uintptr_t)tab2 & 15) || !S || tab_len != LSE_LAST + 1 || fr <= LSE_STEP ||
      fr > 24)
    return BX_EARG;
  if (M == 0) return BX_OK;
  int ch, nch;
  logp_plan(M, V, ch, nch);
  cudaStream_t st = (cudaStream_t)stream;
  i64* psum = (i64*)scratch;
  logp_sum_kernel<<<dim3(nch, M), LOGP_THREADS, 0, st>>>((const i64*)logits, ld, (const i64*)rowmax, nullptr, 0, nullptr,
                                                        (const longlong2*)tab2, psum, V, ch, nch, fr);
  logp_rowfold_kernel<<<(M + 127) / 128, 128, 0, st>>>(psum, nch, (i64*)S, M, 1);
  return launched(2);
}

int bx_logp_finish(const int64_t* S, const int64_t* zt, const int64_t* lnt, int64_t* out, int M, int fr, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!S || !zt || !lnt || !out || M < 0 || fr <= LSE_STEP || fr > 24) return BX_EARG;
  if (M == 0) return BX_OK;
  logp_finish_kernel<<<(M + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const i64*)S, 1, (const i64*)zt, nullptr, 0, nullptr,
                                                                        nullptr, (const i64*)lnt, (i64*)out, M, 0, fr);
  return launched(1);
}

int bx_int_logp(const int64_t* logits, int64_t ld, const int64_t* tok, const int64_t* lnt, const int64_t* tab2,
                int tab_len, void* scratch, int64_t* out, int M, int V, int fr, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!logp_args_ok(logits, ld, scratch, M, V) || !tok || !lnt || !tab2 || ((uintptr_t)tab2 & 15) || !out || tab_len != LSE_LAST + 1 ||
      fr <= LSE_STEP || fr > 24)
    return BX_EARG;
  if (M == 0) return BX_OK;
  int ch, nch;
  logp_plan(M, V, ch, nch);
  cudaStream_t st = (cudaStream_t)stream;
  const int nch0 = sample_chunks(M, V);
  i64* pmax = (i64*)scratch;                       // chunk maxima, then (entry 0 of each row) the row maximum
  i64* psum = pmax + (size_t)M * nch0;
  logp_max_kernel<<<dim3(nch, M), LOGP_THREADS, 0, st>>>((const i64*)logits, ld, pmax, V, ch, nch);
  // the row maxima go to out[], which the last kernel overwrites after reading them
  logp_sum_kernel<<<dim3(nch, M), LOGP_THREADS, 0, st>>>((const i64*)logits, ld, nullptr, pmax, nch, (i64*)out,
                                                        (const longlong2*)tab2, psum, V, ch, nch, fr);
  logp_finish_kernel<<<(M + 127) / 128, 128, 0, st>>>(psum, nch, nullptr, (const i64*)logits, ld, (const i64*)tok,
                                                      (const i64*)out, (const i64*)lnt, (i64*)out, M, V, fr);
  return launched(3);
}

int bx_exact_silu_prod(const int64_t* y, const int64_t* lut, int64_t* P, int64_t* rowmax, int32_t* flag, int N, int FFl,
                       void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !lut || !P || !rowmax || !flag || N < 0 || FFl <= 0) return BX_EARG;
  if (N == 0) return BX_OK;
  silu_prod_kernel<512><<<N, 512, 0, (cudaStream_t)stream>>>((const i64*)y, (const i64*)lut, (i64*)P, (i64*)rowmax, flag,
                                                             FFl);
  return launched(1);
}

int bx_exact_quant_rows(const int64_t* P, const int64_t* rowmax, int fbits, int32_t* q, int64_t ldq, int64_t* sh,
                        int8_t* a8, int64_t plane, int N, int K, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!P || !rowmax || !q || N < 0 || K <= 0 || ldq < K || fbits < 0 || fbits > 62 || (a8 && plane < (int64_t)N * ldq))
    return BX_EARG;
  if (N == 0) return BX_OK;
  quant_rows_kernel<<<N, 256, 0, (cudaStream_t)stream>>>((const i64*)P, (const i64*)rowmax, fbits, q, ldq, (i64*)sh, a8,
                                                         plane, K);
  return launched(1);
}

// ---- stages of the reference's standalone engine, one kernel each (unfused_stages.cuh) ----
int bx_exact_rms(const int64_t* x, int64_t* r, int64_t* er, int64_t* amax, int M, int D, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!x || !r || !er || M < 0 || D < 1 || D > 4096 || (D & (D - 1))) return BX_EARG;
  if (M == 0) return BX_OK;
  int lg = 0;
  while ((1 << lg) < D) ++lg;
  rms_kernel<<<M, US_THREADS, 0, (cudaStream_t)stream>>>((const i64*)x, (i64*)r, (i64*)er, (i64*)amax, D, lg);
  return launched(1);
}

int bx_exact_ndiv(const int64_t* x, const int64_t* gm, const int64_t* ge, const int64_t* r, const int64_t* er,
                  int64_t* P, int M, int D, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!x || !gm || !ge || !r || !er || !P || M < 0 || D < 1) return BX_EARG;
  if (M == 0) return BX_OK;
  ndiv_kernel<<<M, US_THREADS, 0, (cudaStream_t)stream>>>((const i64*)x, (const i64*)gm, (const i64*)ge, (const i64*)r,
                                                        (const i64*)er, (i64*)P, D);
  return launched(1);
}

int bx_rowmax_abs(const int64_t* P, int64_t* rowmax, int M, int K, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!P || !rowmax || M < 0 || K < 1) return BX_EARG;
  if (M == 0) return BX_OK;
  rowmax_abs_kernel<<<M, US_THREADS, 0, (cudaStream_t)stream>>>((const i64*)P, (i64*)rowmax, K);
  return launched(1);
}

int bx_exact_rope(const int64_t* y, const int64_t* cos, const int64_t* sin, const int64_t* pos, int64_t* Pq, int64_t* k,
                  int64_t* v, int N, int H, int HKV, int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!y || !cos || !sin || !pos || !Pq || !k || !v || N < 0 || H <= 0 || HKV <= 0 || HD <= 0 || HD % 2) return BX_EARG;
  if (N == 0) return BX_OK;
  rope_kernel<<<N, US_THREADS, 0, (cudaStream_t)stream>>>((const i64*)y, (const i64*)cos, (const i64*)sin,
                                                        (const i64*)pos, (i64*)Pq, (i64*)k, (i64*)v, H, HKV, HD);
  return launched(1);
}

int bx_softmax_w(const int64_t* raw, const uint8_t* ok, const int64_t* qpos, const int64_t* sh, const int64_t* lut,
                 int64_t l2e, const int32_t* ptab, int32_t* p, int64_t* den, int R, int S, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!raw || !p || !den || R < 0 || S < 1 || (!ok && !qpos)) return BX_EARG;
  if (!ptab && (!sh || !lut)) return BX_EARG;
  if (R == 0) return BX_OK;
  AttnParams w{};
  w.lut = (const i64*)lut;
  w.l2e = (i64)l2e;
  w.ptab = ptab;
  softmax_w_kernel<<<R, US_THREADS, 0, (cudaStream_t)stream>>>((const i64*)raw, ok, (const i64*)qpos,
                                                             ptab ? nullptr : (const i64*)sh, w, p, (i64*)den, S);
  return launched(1);
}

int bx_exact_attn_div(const int64_t* num, const int64_t* den, int64_t* o, int Z, int HD, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!num || !den || !o || Z < 0 || HD < 1) return BX_EARG;
  if (Z == 0) return BX_OK;
  attn_div_kernel<<<Z, US_THREADS, 0, (cudaStream_t)stream>>>((const i64*)num, (const i64*)den, (i64*)o, HD);
  return launched(1);
}

int bx_int8_post_acc(const int64_t* acc, const int64_t* mul, int64_t fmsh, const int64_t* mant, const int64_t* e,
                     int64_t* y, int32_t* flag, int M, int N, int checked, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!acc || !mul || !mant || !e || !y || !flag || M < 0 || N <= 0) return BX_EARG;
  if (M == 0) return BX_OK;
  const int64_t total = (int64_t)M * N;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  i8::int8_post_acc_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const i64*)acc, (const i64*)mul, (i64)fmsh,
                                                                   (const i64*)mant, (const i64*)e, (i64*)y, flag, M, N,
                                                                   checked);
  return launched(1);
}

int bx_pcg_seed_state(const int64_t* keys, int64_t* st, int n, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!keys || !st || n < 0) return BX_EARG;
  if (n == 0) return BX_OK;
  pcg_seed_state_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const i64*)keys, (i64*)st, n);
  return launched(1);
}

int bx_pcg_raw_from_state(const int64_t* st, int64_t* out, int n, int V, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!st || !out || n < 0 || V <= 0) return BX_EARG;
  if (n == 0) return BX_OK;
  const int run = 16;
  const int blocks = (V + run * SAMPLE_THREADS - 1) / (run * SAMPLE_THREADS);
  pcg_raw_state_kernel<<<dim3(blocks, n), SAMPLE_THREADS, 0, (cudaStream_t)stream>>>((const i64*)st, (i64*)out, V, run);
  return launched(1);
}

int bx_bmm(const void* a, int a_is_int64, const void* b, int b_is_int64, int64_t* c, int Z, int M, int N, int K,
           int64_t saz, int64_t sam, int64_t sak, int64_t sbz, int64_t sbk, int64_t sbn, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!a || !b || !c || Z < 0 || M < 0 || N < 0 || K < 0 || K >= 43690 || Z > 65535) return BX_EARG;
  if (Z == 0 || M == 0 || N == 0) return BX_OK;
  const dim3 grid((N + BMM_T - 1) / BMM_T, (M + BMM_T - 1) / BMM_T, Z);
  if (grid.y > 65535) return BX_EARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (a_is_int64 && b_is_int64)
    bmm_kernel<i64, i64><<<grid, 256, 0, st>>>((const i64*)a, (const i64*)b, (i64*)c, M, N, K, saz, sam, sak, sbz, sbk, sbn);
  else if (a_is_int64)
    bmm_kernel<i64, int32_t><<<grid, 256, 0, st>>>((const i64*)a, (const int32_t*)b, (i64*)c, M, N, K, saz, sam, sak, sbz, sbk, sbn);
  else if (b_is_int64)
    bmm_kernel<int32_t, i64><<<grid, 256, 0, st>>>((const int32_t*)a, (const i64*)b, (i64*)c, M, N, K, saz, sam, sak, sbz, sbk, sbn);
  else
    bmm_kernel<int32_t, int32_t><<<grid, 256, 0, st>>>((const int32_t*)a, (const int32_t*)b, (i64*)c, M, N, K, saz, sam, sak, sbz, sbk, sbn);
  return launched(1);
}

// ---- bmm on the tensor pipe (bmm_limb.cuh) ----
size_t bx_bmm_limb_scratch_bytes(int Z, int M, int N, int K) {
  if (Z <= 0 || M < 0 || N < 0 || K < 0) return 0;
  const size_t K16 = ((size_t)K + 15) / 16 * 16;
  return 3 * (size_t)Z * ((size_t)M + (size_t)N) * K16 + 16;
}

int bx_bmm_limb(const void* a, int a_is_int64, const void* b, int b_is_int64, int64_t* c, int Z, int M, int N, int K,
                int64_t saz, int64_t sam, int64_t sak, int64_t sbz, int64_t sbk, int64_t sbn, int8_t* scratch,
                int tile_rows, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (Z < 0 || M < 0 || N < 0 || K < 0 || K >= 43690) return BX_EARG;
  if (Z == 0 || M == 0 || N == 0) return BX_OK;
  if (!c) return BX_EARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (K == 0)                                        // an empty sum (the operands may be null pointers)
    return cudaMemsetAsync(c, 0, sizeof(int64_t) * (size_t)Z * M * N, st) == cudaSuccess ? BX_OK : BX_ELAUNCH;
  if (!a || !b || !scratch || !aligned16(scratch)) return BX_EARG;
  const int K16 = (K + 15) / 16 * 16;
  int8_t* pa = scratch;
  int8_t* pb = scratch + 3 * (size_t)Z * M * K16;
  if (a_is_int64) launch_bmm_pack<i64>(a, saz, sam, sak, pa, Z, M, K, K16, st);
  else launch_bmm_pack<int32_t>(a, saz, sam, sak, pa, Z, M, K, K16, st);
  if (b_is_int64) launch_bmm_pack<i64>(b, sbz, sbn, sbk, pb, Z, N, K, K16, st);      // rows of b^T: columns of b
  else launch_bmm_pack<int32_t>(b, sbz, sbn, sbk, pb, Z, N, K, K16, st);
  int ta = tile_rows;
  if (ta == 0) {
    ta = M <= 16 ? 16 : M <= 32 ? 32 : M <= 48 ? 48 : M <= 64 ? 64 : 80;
    if (M > 80) {
      long best = -1;
      const int cand[3] = {80, 64, 48};
      for (int i = 0; i < 3; ++i) {
        const long cost = (long)((M + cand[i] - 1) / cand[i]) * (cand[i] + 16);
        if (best < 0 || cost < best) { best = cost; ta = cand[i]; }
      }
    }
  }
  CUtensorMap mb, ma;
  if (!make_map(&mb, pb, (uint64_t)K16, (uint64_t)Z * N, 3, WROWS)) return BX_ELAUNCH;
  if (!make_map(&ma, pa, (uint64_t)K16, (uint64_t)Z * M, 3, (uint32_t)ta)) return BX_ELAUNCH;
  BmmEpiParams ep{c, M, N};
  switch (ta) {
    case 16: return launch_bmm_limb<16>(mb, ma, ep, Z, K16, st);
    case 32: return launch_bmm_limb<32>(mb, ma, ep, Z, K16, st);
    case 48: return launch_bmm_limb<48>(mb, ma, ep, Z, K16, st);
    case 64: return launch_bmm_limb<64>(mb, ma, ep, Z, K16, st);
    case 80: return launch_bmm_limb<80>(mb, ma, ep, Z, K16, st);
    default: return BX_EARG;
  }
}

int bx_exact_epilogue(const int64_t* T, const int64_t* B, const int32_t* q, int64_t ldq, const int32_t* cnt,
                      const int32_t* ec, const int64_t* ev, int R, const int64_t* d, const int64_t* g,
                      const int64_t* sh, int64_t* y, int32_t* flag, int M, int N, int checked, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!T || !d || !g || !sh || !y || !flag || M < 0 || N <= 0) return BX_EARG;
  if (cnt && (!q || !ec || !ev || R <= 0)) return BX_EARG;
  if (M == 0) return BX_OK;
  const int64_t total = (int64_t)M * N;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  epilogue_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const i64*)T, (const i64*)B, q, ldq, cnt, ec,
                                                                      (const i64*)ev, R, (const i64*)d, (const i64*)g,
                                                                      (const i64*)sh, (i64*)y, flag, M, N, checked);
  return launched(1);
}

int bx_int8_mm(const int8_t* a, const int8_t* w, int32_t* c, int M, int N, int K, int tile_rows, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!c) return BX_EARG;
  Int8EpiParams ep{c, nullptr, 0, nullptr, nullptr, nullptr, nullptr, M, N, 0};
  return run_int8<false>(a, w, ep, K, tile_rows, (cudaStream_t)stream);
}

int bx_int8_linear_post(const int8_t* a, const int8_t* w, const int64_t* mul, int64_t fmsh, const int64_t* mant,
                        const int64_t* e, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                        void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!mul || !mant || !e || !y || !flag) return BX_EARG;
  Int8EpiParams ep{nullptr, mul, fmsh, mant, e, y, flag, M, N, checked};
  return run_int8<true>(a, w, ep, K, tile_rows, (cudaStream_t)stream);
}

int bx_exact_linear(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                    const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                    int8_t* scratch, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                    void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!q || !sh || !limbs || !d || !g || !scratch || !y || !flag) return BX_EARG;
  if (M < 0 || N <= 0 || K <= 0 || K % 16 || K >= 43690 || !aligned16(limbs) || !aligned16(scratch)) return BX_EARG;
  if (cnt && (!ec || !ev || R <= 0)) return BX_EARG;
  if (M == 0) return BX_OK;
  int rc = bx_split_limbs(q, ldq, scratch, M, K, stream);
  if (rc != BX_OK) return rc;
  return exact_linear_core(q, ldq, sh, limbs, d, g, cnt, ec, ev, R, scratch, y, flag, M, N, K, checked, tile_rows, stream);
}

int bx_exact_linear_planes(const int8_t* planes, const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs,
                           const int64_t* d, const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev,
                           int R, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                           void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (!planes || !sh || !limbs || !d || !g || !y || !flag) return BX_EARG;
  if (M < 0 || N <= 0 || K <= 0 || K % 16 || K >= 43690 || !aligned16(limbs) || !aligned16(planes)) return BX_EARG;
  if (cnt && (!ec || !ev || R <= 0 || !q)) return BX_EARG;
  if (M == 0) return BX_OK;
  return exact_linear_core(q, ldq, sh, limbs, d, g, cnt, ec, ev, R, planes, y, flag, M, N, K, checked, tile_rows, stream);
}

// ---- allocation-free variant of the exact linear ----
// Scratch for the activation limb planes lives in the library image instead of caller memory.
#define BX_STATIC_SCRATCH_BYTES (3u * 256u * 8192u)
static __device__ __align__(256) int8_t g_static_planes[BX_STATIC_SCRATCH_BYTES];

size_t bx_exact_linear_static_max_bytes(void) { return (size_t)BX_STATIC_SCRATCH_BYTES; }

int bx_exact_linear_static(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                           const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                           int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows, void* stream) {
  if (g_status_seen.load(std::memory_order_relaxed)) return BX_EDEVICE;
  if (M < 0 || K <= 0) return BX_EARG;
  if ((size_t)3 * (size_t)M * (size_t)K > (size_t)BX_STATIC_SCRATCH_BYTES) return BX_ELIMIT;
  // The host-side name of a __device__ array is not a device address; resolve it once per device, with that
  // device current, and hand the real address to the kernels.
  // The table is atomic: first calls that race on one device from several host threads store the same address.
  static std::atomic<int8_t*> dev_ptr[BX_MAX_DEVICES];
  const int dev = current_device();
  if (dev < 0) return BX_ELAUNCH;
  int8_t* planes = dev_ptr[dev].load(std::memory_order_acquire);
  if (!planes) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_planes) != cudaSuccess || !p) return BX_ELAUNCH;
    planes = static_cast<int8_t*>(p);
    dev_ptr[dev].store(planes, std::memory_order_release);
  }
  return bx_exact_linear(q, ldq, sh, limbs, d, g, cnt, ec, ev, R, planes, y, flag, M, N, K, checked, tile_rows,
                         stream);
}

}  // extern "C"
