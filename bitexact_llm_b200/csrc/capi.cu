// C ABI of libbitexact_b200.so (declared in include/bitexact_b200.h). One translation unit: the kernel headers
// are included here so that the device-side status word is shared by every kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/bitexact_b200.h"
#include "exact_linear.cuh"

namespace {

using namespace bx;

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

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int TA>
int launch_exact(const CUtensorMap& mw, const CUtensorMap& ma, const ExactEpiParams& ep, int K, cudaStream_t st) {
  using Cfg = GemmCfg<3, 3, TA>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(exact_linear_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) !=
        cudaSuccess)
      return BX_ELAUNCH;
    configured = true;
  }
  const int m_tiles = (ep.M + TA - 1) / TA;
  const int n_tiles = (ep.N + WROWS - 1) / WROWS;
  exact_linear_kernel<TA><<<m_tiles * n_tiles, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(mw, ma, ep, K, m_tiles);
  return cudaGetLastError() == cudaSuccess ? BX_OK : BX_ELAUNCH;
}

}  // namespace

extern "C" {

int bx_version(void) { return 1; }

int bx_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, bx::g_wait_timeouts, sizeof(int)) != cudaSuccess) return BX_ELAUNCH;
  return v;
}

int bx_clear_device_status(void) {
  int v = 0;
  return cudaMemcpyToSymbol(bx::g_wait_timeouts, &v, sizeof(int)) == cudaSuccess ? BX_OK : BX_ELAUNCH;
}

size_t bx_exact_linear_scratch_bytes(int M, int K) { return (size_t)3 * (size_t)M * (size_t)K; }

int bx_split_limbs(const int32_t* q, int64_t ldq, int8_t* a8, int M, int K, void* stream) {
  if (!q || !a8 || M < 0 || K <= 0 || K % 16 || ldq % 4 || ldq < K || !aligned16(q) || !aligned16(a8)) return BX_EARG;
  if (M == 0) return BX_OK;
  const int64_t total = (int64_t)M * (K / 16);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  split_limbs_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, ldq, a8, M, K);
  return cudaGetLastError() == cudaSuccess ? BX_OK : BX_ELAUNCH;
}

int bx_exact_linear(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                    const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                    int8_t* scratch, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                    void* stream) {
  if (!q || !sh || !limbs || !d || !g || !scratch || !y || !flag) return BX_EARG;
  if (M < 0 || N <= 0 || K <= 0 || K % 16 || K >= 43690 || !aligned16(limbs) || !aligned16(scratch)) return BX_EARG;
  if (cnt && (!ec || !ev || R <= 0)) return BX_EARG;
  if (M == 0) return BX_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = bx_split_limbs(q, ldq, scratch, M, K, stream);
  if (rc != BX_OK) return rc;
  int ta = tile_rows;
  if (ta == 0) ta = M <= 16 ? 16 : M <= 32 ? 32 : M <= 48 ? 48 : M <= 64 ? 64 : 80;
  CUtensorMap mw, ma;
  if (!make_map(&mw, limbs, (uint64_t)K, (uint64_t)N, 3, WROWS)) return BX_ELAUNCH;
  if (!make_map(&ma, scratch, (uint64_t)K, (uint64_t)M, 3, (uint32_t)ta)) return BX_ELAUNCH;
  ExactEpiParams ep{q, ldq, sh, d, g, cnt, ec, ev, R, y, flag, M, N, checked};
  switch (ta) {
    case 16: return launch_exact<16>(mw, ma, ep, K, st);
    case 32: return launch_exact<32>(mw, ma, ep, K, st);
    case 48: return launch_exact<48>(mw, ma, ep, K, st);
    case 64: return launch_exact<64>(mw, ma, ep, K, st);
    case 80: return launch_exact<80>(mw, ma, ep, K, st);
    default: return BX_EARG;
  }
}

}  // extern "C"
