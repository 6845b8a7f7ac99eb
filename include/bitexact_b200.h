/* C ABI of libbitexact_b200.so: hand-written sm_100a kernels for the integer hot path of the bit-exact
 * Llama engine. Plain pointers and sizes only; every pointer is a DEVICE pointer unless said otherwise.
 * All entry points return 0 on success and a negative BX_E* code on an argument or launch error. Arithmetic
 * bound violations never raise: kernels set the caller's sticky `flag` word to 1 (it is never cleared).
 * `stream` is a cudaStream_t passed as void* (NULL = default stream). Calls are asynchronous.
 *
 * Each declaration cites the reference interface it replaces (paths inside mynotwo/bitexact-llm).
 */
#ifndef BITEXACT_B200_H
#define BITEXACT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BX_OK 0
#define BX_EARG (-1)     /* shape / alignment / null-pointer contract violated */
#define BX_ELAUNCH (-2)  /* CUDA launch or driver call failed */
#define BX_EDEVICE (-3)  /* a bounded device-side wait gave up (see bx_device_status) */

/* Library / device state. bx_device_status: number of device-side waits that timed out since the last clear
 * (0 in a healthy run; synchronises the device). */
int bx_version(void);
int bx_device_status(void);
int bx_clear_device_status(void);

/* ---- exact-mode linear -------------------------------------------------------------------------------
 * y[m, n] = round((sum_k q[m, k] W[n, k] * 2^d[n] + B[m, n]) * 2^(sh[m] + g[n] - d[n] + 24)), one rounding,
 * W = limbs[0] + 256 limbs[1] + 65536 limbs[2], B = sparse residual in padded per-row (ELL) form.
 * Replaces FusedLin.__call__ (src/bitexact/vllm_plugin/exact_gemm.py:284-316; kernel :58-119), i.e.
 * wmm + residual + epilogue of src/bitexact/exact/wmm.py:79-150.
 *   q      int32 [M, K], row stride ldq elements (ldq % 4 == 0, 16-byte aligned), |q| <= 2^22
 *   sh     int64 [M]
 *   limbs  int8 [3, N, K] contiguous (16-byte aligned), K % 16 == 0, K < 43690
 *   d, g   int64 [N]
 *   cnt    int32 [N] residual entries per row, ec int32 [N, R] columns, ev int64 [N, R] values (cnt NULL: none)
 *   scratch  int8, bx_exact_linear_scratch_bytes(M, K) bytes, 16-byte aligned (activation limb planes)
 *   y      int64 [M, N] contiguous;  flag int32 [1], set to 1 when `checked` and a result lost bits or left
 *          (-2^62, 2^62)
 *   tile_rows  activation rows per CTA tile: 0 = automatic, else one of 16, 32, 48, 64, 80 (no effect on results)
 */
size_t bx_exact_linear_scratch_bytes(int M, int K);
int bx_exact_linear(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                    const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                    int8_t* scratch, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                    void* stream);

/* Activation limb planes only: q int32 [M, K] -> a8 int8 [3, M, K] (signed base-256 digits,
 * src/bitexact/intops.py:62-70). */
int bx_split_limbs(const int32_t* q, int64_t ldq, int8_t* a8, int M, int K, void* stream);

#ifdef __cplusplus
}
#endif
#endif
