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
#define BX_ELIMIT (-4)   /* the request exceeds a fixed capacity of the entry point (see its comment) */

/* Library / device state. Every device-side wait of the kernels is bounded; one that gives up adds 1 to a status
 * word on the device, and from then on every CTA of the pipelined kernels returns at once WITHOUT writing its
 * outputs (the word is sticky). The reference has no counterpart: its Triton kernels have no waits of their own.
 *   bx_device_status        the word (0 in a healthy run); copies it from the device, which synchronises.
 *   bx_clear_device_status  back to 0.
 *   bx_set_device_status    writes the word from the host (value >= 0): lets a host application or a test put the
 *                           device into the failed state without making any wait run out on it.
 * Launching entry points do not read the word themselves (that would synchronise every launch). Once the host has
 * SEEN a non-zero word (bx_device_status returned it) every launching entry point returns BX_EDEVICE and
 * launches nothing, until bx_clear_device_status. The engines' check() reads the
 * word. Kernel attributes and device properties are cached per device ordinal (up to 64 devices per process). */
int bx_version(void);
long long bx_launch_count(void);   /* kernels launched through this library so far (host-side count) */
int bx_device_status(void);
int bx_clear_device_status(void);
int bx_set_device_status(int value);

/* Measured int8 tensor-pipe peak of the current device (a measurement utility; no counterpart in the reference):
 * one CTA per SM issues tcgen05.mma kind::i8 (M 128, N 256, K 32) `iters` x 4 times on operands resident in shared
 * memory (no TMA, no global memory, no epilogue in the loop); `repeats` timed launches after a warm-up one.
 * tops (HOST pointer, double [2]) receives the best and the mean rate in int8 TOPS (2 ops per multiply-add).
 * Synchronises the stream. iters 4 .. 2^22 (2^17 runs about 5 ms on a B200), repeats 1 .. 64. */
int bx_i8_tensor_peak(int iters, int repeats, double* tops, void* stream);

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
 *   tile_rows  activation rows per CTA tile: 0 = automatic, else one of 16, 32, 48, 64, 80; -16, -32, -48 select
 *              that tile size on the persistent kernel (one CTA per SM, overlapped epilogue); 216, 232, 264 select
 *              16, 32, 64 rows with the K dimension split over a cluster of up to 8 CTAs (partial sums through
 *              distributed shared memory), the automatic choice for M <= 128 when the tile list covers less than
 *              half of the SMs (10000 S + 2xx: clusters of exactly S = 2, 4 or 8 CTAs); 416, 432, 448: that many
 *              activation rows on CTA pairs (tcgen05 cta_group::2, 256 weight rows per pair); 516 .. 580 and
 *              616 .. 680 (steps of 16): the ACTIVATION rows on the MMA M side and that many weight rows per tile,
 *              on CTA pairs / on one CTA (the automatic choice for long tile lists of batches of 128 rows and
 *              more: 664); 764 (10000 S + 764): 64 weight rows per tile with the activation rows on the M side and
 *              K split over clusters of S = 2 or 4 CTAs (the automatic choice for short tile lists with K >= 8192
 *              at 128 rows and more). No effect on results.
 */
size_t bx_exact_linear_scratch_bytes(int M, int K);
int bx_exact_linear(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                    const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                    int8_t* scratch, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                    void* stream);

/* bx_exact_linear when the activation limb planes already exist (the stage kernels bx_exact_norm,
 * bx_exact_attn_out and bx_exact_silu_quant write them next to q through their `a8` argument): no splitting pass,
 * no scratch. planes int8 [3, M, K], 16-byte aligned; q (only read for the sparse residual) may be NULL when cnt is
 * NULL. Same results as bx_exact_linear. */
int bx_exact_linear_planes(const int8_t* planes, const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs,
                           const int64_t* d, const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev,
                           int R, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                           void* stream);

/* bx_exact_linear for callers that must not allocate device memory. It has no counterpart in the reference.
 *
 * Some hosts of this library cannot provide the scratch buffer bx_exact_linear asks for: a plugin that is
 * invoked while its host application is recording a CUDA graph or has frozen its memory pool, a runtime with a
 * fixed arena and no allocator behind it, a service that forbids cudaMalloc after start-up to keep latency flat.
 * For them the activation limb planes go into a fixed buffer that is part of the library image
 * (bx_exact_linear_static_max_bytes() = 3 * 256 * 8192 bytes = 6 MiB; every GPU that loads the library keeps it
 * until the process exits). Same arguments as bx_exact_linear without `scratch`; same results bit for bit.
 *   - 3 * M * K must not exceed the buffer: larger requests return BX_ELIMIT and launch nothing.
 *   - The first call on each device looks up the buffer's device address (one driver query, no allocation);
 *     make that first call during start-up, before any stream capture begins. First calls may come from
 *     several host threads at once: the address table is atomic and they all store the same value.
 *   - The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - All calls on a device share the one buffer and it keeps the previous call's contents. Nothing in it has to
 *     start at zero (each call overwrites every byte it later reads), but two calls that run on the GPU at the
 *     same time - different streams, or different host threads - race on it: serialise them on one stream. */
size_t bx_exact_linear_static_max_bytes(void);
int bx_exact_linear_static(const int32_t* q, int64_t ldq, const int64_t* sh, const int8_t* limbs, const int64_t* d,
                           const int64_t* g, const int32_t* cnt, const int32_t* ec, const int64_t* ev, int R,
                           int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows, void* stream);

/* ---- int8-mode linear ----------------------------------------------------------------------------------
 * a: the two activation limbs stacked along rows as the reference's stack_limbs(q, 2) lays them out
 * (src/bitexact/intops.py:73-79): int8 [R, K], limb i of row m at row i * M + m (R >= 2 M; rows beyond 2 M are
 * padding and are not read). w: int8 [N, K]. Both 16-byte aligned, K % 16 == 0.
 *
 * bx_int8_mm: c int32 [R, N]: rows [0, M) = limb-0 products, rows [M, 2 M) = limb-1 products (padding rows are
 * not written). Replaces int_mm (src/bitexact/int8/gemm_skinny.py:80-97; CPU: imm, src/bitexact/int8/ops.py:87-90).
 *
 * bx_int8_linear_post: the same product with segs.post fused (src/bitexact/int8/segs.py:62-67; fused copy
 * tri_fuse._y, src/bitexact/vllm_plugin/tri_fuse.py:74-79): acc = c0 + (c1 << 8); t = rsh(acc * mul[n], fmsh);
 * y[m, n] = rsh(t * mant[m], 8 - e[m]) at 16 fractional bits; flag set when `checked` and some |t| >= 2^38.
 * tile_rows: 0 = automatic, else 16, 32, 64 or 128; -16 .. -128 select that tile size on the persistent kernel (one
 * CTA per SM, two accumulator buffers), the automatic choice when there are more tiles than SMs; for
 * bx_int8_linear_post also 216, 232, 264 (10000 S + 2xx: clusters of exactly S = 2, 4 or 8): that many rows per tile
 * with the K dimension split over a cluster of CTAs, the automatic choice when the tile list covers less than half
 * of the SMs. No effect on results. */
int bx_int8_mm(const int8_t* a, const int8_t* w, int32_t* c, int M, int N, int K, int tile_rows, void* stream);
int bx_int8_linear_post(const int8_t* a, const int8_t* w, const int64_t* mul, int64_t fmsh, const int64_t* mant,
                        const int64_t* e, int64_t* y, int32_t* flag, int M, int N, int K, int checked, int tile_rows,
                        void* stream);

/* Activation limb planes only: q int32 [M, K] -> a8 int8 [3, M, K] (signed base-256 digits,
 * src/bitexact/intops.py:62-70). */
int bx_split_limbs(const int32_t* q, int64_t ldq, int8_t* a8, int M, int K, void* stream);

/* ---- exact-mode element-wise stages (one launch each) ---------------------------------------------------
 * Shared conventions: rows are independent; `flag` is the sticky int32 bound flag; `a8` (may be NULL) receives
 * the int8 limb planes [3, M, K] of the quantised row q next to q itself, so a following bx_exact_linear_planes
 * call needs no splitting pass.
 */

/* RMSNorm + power-of-two quantisation. mode 0: x = emb[ids[m]] (emb int32 [V, D]); 1: x = xin + yin; 2: x = xin
 * (int64 [M, D]). xo (may be NULL) receives x. With do_norm: q int32 [M, D], sh int64 [M] of
 * quant(div_round(x * gamma, ...), -40); gm / ge int64 [D] are gamma's exact bf16 significand and exponent.
 * D a power of two, 32 <= D <= 4096. Sets flag when max |x| >= 2^40.
 * Replaces exact_fuse.embed_norm / add_norm / pre_norm (src/bitexact/vllm_plugin/exact_fuse.py:136-175, 342-373)
 * = segs.add_y + Segs.norm_q (src/bitexact/exact/segs.py:44-68, 150-155). */
int bx_exact_norm(int mode, const void* xin, const int64_t* yin, const int64_t* ids, const int64_t* gm,
                  const int64_t* ge, int64_t* xo, int32_t* q, int64_t* sh, int8_t* a8, int32_t* flag, int M, int D,
                  int do_norm, void* stream);

/* RoPE (30-bit cos / sin) of q and k, v >> 5, per-(token, head) quantisation of q, K / V limb planes stored at
 * `slot` of the paged cache (cache NULL: no store; slot < 0: token skipped).
 *   y int64 [N, (H + 2 HKV) HD] at 24 bits; cos, sin int64 [max_pos, HD / 2]; pos, slot int64 [N]
 *   cache int8 [nb, HKV, bs, 8 HD] with element strides sc_nb, sc_h, sc_bs (last dimension contiguous)
 *   q int32 [N, H HD], sh int64 [N, H].  HD in {64, 128}.
 * Replaces exact_fuse.qkv (src/bitexact/vllm_plugin/exact_fuse.py:178-236, 376-391) = segs.rope_y + q_group
 * (src/bitexact/exact/segs.py:78-99) + tri_paged.store. */
int bx_exact_qkv(const int64_t* y, const int64_t* cos, const int64_t* sin, const int64_t* pos,
                 const int64_t* slot, int8_t* cache, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, int32_t* q,
                 int64_t* sh, int32_t* flag, int N, int H, int HKV, int HD, void* stream);

/* K / V int64 [N, HKV, HD] (element strides skz, skh / svz, svh) -> limb planes at flat slots.
 * Replaces tri_paged.store (src/bitexact/vllm_plugin/tri_paged.py:311-335). */
int bx_kv_store(int8_t* cache, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const int64_t* slot,
                const int64_t* k, int64_t skz, int64_t skh, const int64_t* v, int64_t svz, int64_t svh, int N,
                int HKV, int HD, void* stream);

/* o = div_round(num, 5, den) per head, then row quantisation at 24 bits. num int64 [N, K2], den int64
 * [N, K2 / HD]; q int32 [N, K2], sh int64 [N]. K2 <= 4096.
 * Replaces exact_fuse.attn_out (src/bitexact/vllm_plugin/exact_fuse.py:239-248, 394-404) = segs.attn_div + quant. */
int bx_exact_attn_out(const int64_t* num, const int64_t* den, int32_t* q, int64_t* sh, int8_t* a8, int N, int K2,
                      int HD, void* stream);

/* silu(gate) * up and row quantisation at 48 bits. y int64 [N, 2 FF] (gate | up), lut = 2^-f table int64 [16385]
 * at 2^60; q int32 [N, FF], sh int64 [N]. FF <= 14336. Sets flag on the reference's product-bound violation.
 * Replaces exact_fuse.silu_quant (src/bitexact/vllm_plugin/exact_fuse.py:266-309, 407-414) = segs.silu_y +
 * quant_silu, ops.silu_mul (src/bitexact/exact/ops.py:119-130). */
int bx_exact_silu_quant(const int64_t* y, const int64_t* lut, int32_t* q, int64_t* sh, int8_t* a8, int32_t* flag,
                        int N, int FF, void* stream);

/* SiLU * up + quantisation in two steps, for a gate / up projection sharded by output column over several GPUs (the
 * reference is single-GPU; same integers as exact_fuse.silu_quant, src/bitexact/vllm_plugin/exact_fuse.py:266-309,
 * 407-414, on the full row). bx_exact_silu_prod: y int64 [N, 2 FFl] (the rank's gate columns, then its up columns)
 * -> P int64 [N, FFl] and rowmax int64 [N] = max |P| over the rank's columns. The caller takes the integer maximum
 * of rowmax over the ranks (an exact all-reduce MAX). bx_exact_quant_rows: q = rshc(P, sh + fbits) with
 * sh = quant_sh(rowmax, -fbits) (src/bitexact/exact/ops.py:82-89; fbits = 48 after SiLU): q int32 with row pitch
 * ldq, sh int64 [N] (may be NULL), optional limb planes a8 (plane = elements per plane, row pitch ldq). */
int bx_exact_silu_prod(const int64_t* y, const int64_t* lut, int64_t* P, int64_t* rowmax, int32_t* flag, int N, int FFl,
                       void* stream);
int bx_exact_quant_rows(const int64_t* P, const int64_t* rowmax, int fbits, int32_t* q, int64_t ldq, int64_t* sh,
                        int8_t* a8, int64_t plane, int N, int K, void* stream);

/* ---- exact-mode paged attention -------------------------------------------------------------------------
 * q int32 [R, HKV, M, 64] (M <= 4), sh int64 [R, HKV, M], qpos int64 [R, M] (key s visible to row i iff
 * s <= qpos[r, i]), cache int8 limb planes [nb, HKV, bs, 512], bt [*, nblk] block table (int32, or int64 when
 * bt_is_int64) with row stride sbt, rmap int64 [R] block-table row per request (NULL: identity), lut = 2^-f table,
 * l2e = round(log2(e) * 2^28) for head_dim 64. Outputs num int64 [R, HKV, M, 64], den int64 [R, HKV, M].
 * nb = number of cache blocks. nblk * bs < 43690. cluster_size: CTAs per (request, head) splitting the keys,
 * 0 = automatic, else 1, 2, 4 or 8. variant: 0 = automatic, 1 = direct-load kernel (any page size / strides),
 * 2 = TMA-staged kernel, 3 / 4 = TMA-staged kernel with p.V on tcgen05 / TMEM and 8 / 4 consumer warps per CTA
 * (2..4: page size 8..64 dividing 64, 16-byte aligned strides; 4: page size <= 32). None of them changes a result.
 * Replaces tri_exact_attn.attend (src/bitexact/vllm_plugin/tri_exact_attn.py:138-165). */
int bx_exact_attention(const int32_t* q, const int64_t* sh, const int64_t* qpos, const int8_t* cache, int64_t nb,
                       int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64,
                       int64_t sbt, int nblk, const int64_t* rmap, const int64_t* lut, int64_t l2e, int64_t* num,
                       int64_t* den, int R, int HKV, int M, int HD, int cluster_size, int variant, void* stream);

/* The same with a scratch buffer (no counterpart in the reference, whose kernels re-read K instead): with scratch of
 * bx_attention_scratch_bytes(nblk, bs) bytes, 16-byte aligned, the persistent streaming kernel also serves contexts
 * whose scores do not fit in shared memory (it keeps them in the scratch, one slice per CTA, and runs its second sweep
 * in chunks of 512 keys). The buffer carries nothing between calls. NULL scratch = bx_exact_attention. */
size_t bx_attention_scratch_bytes(int nblk, int bs);
int bx_exact_attention_ws(const int32_t* q, const int64_t* sh, const int64_t* qpos, const int8_t* cache, int64_t nb,
                          int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64,
                          int64_t sbt, int nblk, const int64_t* rmap, const int64_t* lut, int64_t l2e, int64_t* num,
                          int64_t* den, int R, int HKV, int M, int HD, int cluster_size, int variant, void* scratch,
                          size_t scratch_bytes, void* stream);
int bx_int8_attention_ws(const int32_t* q, const int64_t* qpos, const int8_t* cache, int64_t nb, int64_t sc_nb,
                         int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64, int64_t sbt, int nblk,
                         const int64_t* rmap, const int32_t* ptab, int64_t* num, int64_t* den, int R, int HKV, int M,
                         int HD, int cluster_size, int variant, void* scratch, size_t scratch_bytes, void* stream);

/* ---- prefill attention (both weight rules) -------------------------------------------------------------------------
 * Attention of whole TILES of prompt tokens: a tile is up to tile_rows / G consecutive tokens of one request; one CTA
 * per (tile, KV head) stages every K / V row once for the tile's query rows (token x G query heads), runs both integer
 * sweeps and has the limb products (scores and p.V) on tcgen05 with TMEM accumulators. tile_rows: 32 (one CTA of
 * 512 threads per SM; 0 selects it) or 16 (two CTAs of 256 threads per SM). No effect on results.
 *   q      int32 [N, HKV, G, 64] token-major (|q| <= 2^22 exact mode; within three limbs int8 mode), 16-byte aligned
 *   sh     int64 [N, HKV, G] row exponents (exact mode; NULL with ptab)
 *   pos    int64 [N] position of each token: key s is visible iff s <= pos
 *   tiles  int32 [n_tiles, 3] = (block-table row, first token, tokens <= tile_rows / G), on the device
 *   cache, bt, nblk, bs as bx_exact_attention (bs one of 8, 16, 32, 64, 128); lut / l2e: exact weight rule;
 *   ptab: int8-mode weight table (then lut may be NULL)
 *   num int64 [N, HKV, G, 64], den int64 [N, HKV, G]: the rows of the tiles' tokens are written, others untouched.
 * Same integers as the per-row kernels on each token. Replaces tri_prefill.attend + tile_table
 * (src/bitexact/vllm_plugin/tri_prefill.py:32-108, int8 weight rule); exact mode has no multi-token kernel in the
 * reference (its plugin runs prompt tokens as rows, src/bitexact/vllm_plugin/exact_run.py:3-7): there the unfused
 * bmm + softmax_w + bmm of src/bitexact/exact/model.py:114-119 is the rule. */
int bx_prefill_attention(const int32_t* q, const int64_t* sh, const int64_t* pos, const int32_t* tiles, int n_tiles,
                         const int8_t* cache, int64_t nb, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs,
                         const void* bt, int bt_is_int64, int64_t sbt, int nblk, const int64_t* lut, int64_t l2e,
                         const int32_t* ptab, int64_t* num, int64_t* den, int HKV, int G, int HD, int tile_rows,
                         void* stream);

/* ---- int8-mode attention and element-wise stages -------------------------------------------------------
 * Fixed points of int8 mode: residual stream / linear outputs / logits 16 bits, gamma 12, cos / sin 16, q / k / v 14,
 * attention weights 20. A linear's input is always (a8, mant, e): activation limb planes int8 [2, M, K] (limb i of
 * row m at row i * M + m: the reference's stack_limbs layout without padding rows) plus the row scale
 * mant * 2^e with mant in [2^23, 2^24]; its output y is the int64 tensor of bx_int8_linear_post.
 */

/* Paged attention with the int8-mode weight rule (direct e^z table, no interpolation, head_dim 64):
 * q int32 [R, HKV, M, 64] (|q| within 3 limbs), ptab int32 [131073] = rsh(exp table, 10); the other arguments as
 * bx_exact_attention. Replaces tri_paged.attend (src/bitexact/vllm_plugin/tri_paged.py:363-430). */
int bx_int8_attention(const int32_t* q, const int64_t* qpos, const int8_t* cache, int64_t nb, int64_t sc_nb,
                      int64_t sc_h, int64_t sc_bs, int bs, const void* bt, int bt_is_int64, int64_t sbt, int nblk,
                      const int64_t* rmap, const int32_t* ptab, int64_t* num, int64_t* den, int R, int HKV, int M,
                      int HD, int cluster_size, int variant, void* stream);

/* x = emb[ids] (mode 0) | xin + yin (mode 1) | xin (mode 2); with do_norm: pre_norm(x, gamma) -> (a8, mant, e),
 * else the |x| >= 2^42 bound flag. gamma int64 [D] at 12 bits. D <= 4096.
 * Replaces tri_fuse.embed_norm / add_norm (src/bitexact/vllm_plugin/tri_fuse.py:82-160) = segs.pre_norm
 * (src/bitexact/int8/segs.py:48-53) after post + residual add. */
int bx_int8_norm(int mode, const void* xin, const int64_t* yin, const int64_t* ids, const int64_t* gamma,
                 int64_t* xo, int8_t* a8, int64_t* mant, int64_t* e, int32_t* flag, int M, int D, int do_norm,
                 void* stream);

/* RoPE (16-bit tables) of q and k, v >> 2, LIM3 bound flag, K / V limb planes stored at `slot` of the paged cache.
 * y int64 [N, (H + 2 HKV) HD]; q64 int64 and / or q32 int32 [N, HKV, G, HD] (either may be NULL).
 * Replaces tri_fuse.qkv (src/bitexact/vllm_plugin/tri_fuse.py:163-214) = segs.qkv (src/bitexact/int8/segs.py:69-88). */
int bx_int8_qkv(const int64_t* y, const int64_t* cos, const int64_t* sin, const int64_t* pos, const int64_t* slot,
                int8_t* cache, int64_t sc_nb, int64_t sc_h, int64_t sc_bs, int bs, int64_t* q64, int32_t* q32,
                int32_t* flag, int N, int H, int HKV, int HD, void* stream);

/* o = rdiv(num << 2, den) per head, pre_plain(o) -> (a8, mant, e). num int64 [N, K2], den int64 [N, K2 / HD].
 * Replaces tri_fuse.attn_out (src/bitexact/vllm_plugin/tri_fuse.py:217-240) = segs.attn_out
 * (src/bitexact/int8/segs.py:101-109). */
int bx_int8_attn_out(const int64_t* num, const int64_t* den, int8_t* a8, int64_t* mant, int64_t* e, int N, int K2,
                     int HD, void* stream);

/* h = rsh(silu_table(gate) * up, 16), pre_plain(h) -> (a8, mant, e). y int64 [N, 2 FF], lut = SiLU table int64
 * [262145]. scr (may be NULL) int64 [2]: receives atomic maxima of |silu(gate)| and |up| for the product-bound flag.
 * Replaces tri_mlp.silu_quant (src/bitexact/vllm_plugin/tri_mlp.py:153-183) = segs.silu_mul
 * (src/bitexact/int8/segs.py:111-118). bx_int8_flag_end: flag |= scr[i][0] * scr[i][1] >= 2^62 for i < L, then
 * clears scr (tri_fuse.flag_end, src/bitexact/vllm_plugin/tri_fuse.py:248-265). */
int bx_int8_silu_quant(const int64_t* y, const int64_t* lut, int8_t* a8, int64_t* mant, int64_t* e, int64_t* scr,
                       int N, int FF, void* stream);
int bx_int8_flag_end(int64_t* scr, int32_t* flag, int L, void* stream);

/* h = rsh(silu_table(gate) * up, 16) and pre_plain(h) in two steps, for a gate / up projection sharded by output column
 * over several GPUs (the reference is single-GPU; same integers as tri_mlp.silu_quant,
 * src/bitexact/vllm_plugin/tri_mlp.py:153-183, on the full row). bx_int8_silu_prod: y int64 [N, 2 FFl] (the rank's gate
 * columns, then its up columns) -> h int64 [N, FFl] and rowmax int64 [N] = max |h| over the rank's columns; scr as in
 * bx_int8_silu_quant. The caller takes the integer maximum of rowmax (and of scr) over the ranks.
 * bx_int8_quant_rows: pre_plain of the rows of h [N, K] with the maxima of the full rows: limb planes a8 [2][N][K] and
 * (mant, e) int64 [N] (may be NULL: every rank computes the same values). */
int bx_int8_silu_prod(const int64_t* y, const int64_t* lut, int64_t* h, int64_t* rowmax, int64_t* scr, int N, int FFl,
                      void* stream);
int bx_int8_quant_rows(const int64_t* h, const int64_t* rowmax, int8_t* a8, int64_t* mant, int64_t* e, int N, int K,
                       void* stream);

/* segs.post on a raw bx_int8_mm output (src/bitexact/int8/segs.py:62-67): c int32 [>= 2 M, N] -> y int64 [M, N].
 * For callers that keep the reference's two-step int_mm + post form; bx_int8_linear_post does both in one kernel. */
int bx_int8_post(const int32_t* c, const int64_t* mul, int64_t fmsh, const int64_t* mant, const int64_t* e, int64_t* y,
                 int32_t* flag, int M, int N, int checked, void* stream);

/* ---- unfused entry points of the reference's standalone engine -------------------------------------------
 * bx_bmm replaces bmm(a, b, na, nb) (src/bitexact/bmm.py:78-102): c[z] = a[z] @ b[z] exactly, a [Z, M, K] and
 * b [Z, K, N] int32 or int64 with element strides (any layout), c int64 [Z, M, N] contiguous; operands of at most
 * three limbs (|x| < 2^23) and K < 43690, so that no sum leaves int64.
 * bx_exact_epilogue replaces segs.lin_y on a dense product (src/bitexact/exact/segs.py:25-32,
 * exact/wmm.py:132-150): y = round((T 2^d + B) 2^(sh + g - d + 24)) with the lost-bit / range flag; B is a dense
 * int64 [M, N] residual (NULL: zero) and / or the ELL residual (cnt, ec, ev as in bx_exact_linear) gathered from q.
 * The dense product T itself (wmm_triton, exact/wmm.py:31-96) is bx_exact_linear with d = 0, g = -24, sh = 0 and no
 * residual: then y = T. */
int bx_bmm(const void* a, int a_is_int64, const void* b, int b_is_int64, int64_t* c, int Z, int M, int N, int K,
           int64_t saz, int64_t sam, int64_t sak, int64_t sbz, int64_t sbk, int64_t sbn, void* stream);
/* The same product on the tensor pipe, the way the reference's Triton kernel forms it (src/bitexact/bmm.py:27-75:
 * up to 3 x 3 int8 limb products into five int32 accumulators, one int64 join at the end): a pass packs both
 * operands into K-major limb planes (b transposed on the way) in `scratch` (bx_bmm_limb_scratch_bytes bytes, 16-byte
 * aligned), then one CTA per (batch, 128 columns of b, tile_rows rows of a) runs the tcgen05 limb main loop.
 * tile_rows: 0 = automatic, else 16, 32, 48, 64 or 80. Same contract and integers as bx_bmm (|x| < 2^23). */
size_t bx_bmm_limb_scratch_bytes(int Z, int M, int N, int K);
int bx_bmm_limb(const void* a, int a_is_int64, const void* b, int b_is_int64, int64_t* c, int Z, int M, int N, int K,
                int64_t saz, int64_t sam, int64_t sak, int64_t sbz, int64_t sbk, int64_t sbn, int8_t* scratch,
                int tile_rows, void* stream);
int bx_exact_epilogue(const int64_t* T, const int64_t* B, const int32_t* q, int64_t ldq, const int32_t* cnt,
                      const int32_t* ec, const int64_t* ev, int R, const int64_t* d, const int64_t* g,
                      const int64_t* sh, int64_t* y, int32_t* flag, int M, int N, int checked, void* stream);

/* ---- stages of the standalone exact engine, one kernel each ------------------------------------------------------
 * The serving path fuses these into bx_exact_norm / bx_exact_qkv / bx_exact_attention / bx_exact_attn_out; the
 * separate forms keep code written against bitexact.exact.segs and bitexact.exact.ops running stage by stage.
 *   bx_exact_rms       ops.rms (src/bitexact/exact/ops.py:92-105): x int64 [M, D] (D a power of two <= 4096) ->
 *                      r, er int64 [M] with sqrt(mean(x^2) + 1e-5) = r 2^er; amax (may be NULL) = max |x| per row.
 *   bx_exact_ndiv      segs.ndiv (src/bitexact/exact/segs.py:49-51): P = div_round(x gm, ge - 24 - er + 40, r).
 *   bx_rowmax_abs      max |P| per row: with bx_exact_quant_rows it is ops.quant (exact/ops.py:82-89).
 *   bx_exact_rope      segs.rope_y (exact/segs.py:78-87) without the quantisation: y int64 [N, (H + 2 HKV) HD] ->
 *                      Pq int64 [N, H, HD] at 54 bits, k [N, HKV, HD] at 17 bits, v [N, HKV, HD] at 19 bits.
 *   bx_softmax_w       ops.softmax_w (exact/ops.py:133-143) on dense scores raw int64 [R, S]: key s of row r takes
 *                      part iff ok[r, s] != 0 (ok uint8 [R, S]) or, with ok NULL, s <= qpos[r]; sh int64 [R] row
 *                      exponents, lut / l2e as bx_exact_attention; with ptab the int8-mode rule
 *                      (int8/segs.py:91-99). p int32 [R, S] (0 where masked), den int64 [R].
 *   bx_exact_attn_div  segs.attn_div (exact/segs.py:108-113): o[z, :] = div_round(num[z, :], 5, den[z]), num int64 [Z, HD].
 *   bx_int8_post_acc   segs.post (int8/segs.py:62-67) on the joined accumulator acc int64 [M, N].
 *   bx_pcg_seed_state / bx_pcg_raw_from_state   gpu_pcg.seed_state / raw_from_state
 *                      (src/bitexact/vllm_plugin/gpu_pcg.py:44-52, 94-104): keys int64 [n, 2] -> st int64 [n, 4]
 *                      (state hi, lo, increment hi, lo after numpy's seeding); st -> raw words int64 [n, V]. */
int bx_exact_rms(const int64_t* x, int64_t* r, int64_t* er, int64_t* amax, int M, int D, void* stream);
int bx_exact_ndiv(const int64_t* x, const int64_t* gm, const int64_t* ge, const int64_t* r, const int64_t* er,
                  int64_t* P, int M, int D, void* stream);
int bx_rowmax_abs(const int64_t* P, int64_t* rowmax, int M, int K, void* stream);
int bx_exact_rope(const int64_t* y, const int64_t* cos, const int64_t* sin, const int64_t* pos, int64_t* Pq, int64_t* k,
                  int64_t* v, int N, int H, int HKV, int HD, void* stream);
int bx_softmax_w(const int64_t* raw, const uint8_t* ok, const int64_t* qpos, const int64_t* sh, const int64_t* lut,
                 int64_t l2e, const int32_t* ptab, int32_t* p, int64_t* den, int R, int S, void* stream);
int bx_exact_attn_div(const int64_t* num, const int64_t* den, int64_t* o, int Z, int HD, void* stream);
int bx_int8_post_acc(const int64_t* acc, const int64_t* mul, int64_t fmsh, const int64_t* mant, const int64_t* e,
                     int64_t* y, int32_t* flag, int M, int N, int checked, void* stream);
int bx_pcg_seed_state(const int64_t* keys, int64_t* st, int n, void* stream);
int bx_pcg_raw_from_state(const int64_t* st, int64_t* out, int n, int V, void* stream);

/* ---- integer sampler ------------------------------------------------------------------------------------
 * Raw PCG64 words of numpy's default_rng([20261022, seed, t]): keys int64 [n, 2] -> out int64 [n, V].
 * Replaces gpu_pcg.raw_rows (src/bitexact/vllm_plugin/gpu_pcg.py:94-108; CPU: src/bitexact/sampling.py:27-37). */
int bx_pcg_raw(const int64_t* keys, int64_t* out, int n, int V, void* stream);

/* Token per row: rows int64 [M, 4] = (seed, t, tn, td); tn == 0 -> first argmax of the logits row, else first
 * argmax of round(l * td / tn) + gumbel(seed, t) at `bits` fractional bits. logits int64 [M, V], row stride ld;
 * lnt = ln table int64 [65537] at 40 bits; scratch: bx_sample_scratch_bytes(M, V) bytes; tok int64 [M].
 * Replaces sampler.integer_sample / tri_logits.first_argmax (src/bitexact/vllm_plugin/sampler.py:57-88,
 * vllm_plugin/tri_logits.py:77-100) = sampling.sample(gumbel(raw_rows(.))) (src/bitexact/sampling.py:50-67). */
/* bx_sample_shard: the same pass over a COLUMN SHARD of the logits (vocabulary entries v_offset .. v_offset +
 * V_local - 1; the noise of entry i is word i of the row's PCG64 stream whatever the shard). Writes per row the
 * shard's maximum `best` and its first global index `idx`; the caller all-gathers the pairs and keeps, per row,
 * the larger `best`, then the smaller `idx` - the rule of the reference's chunk combine
 * (src/bitexact/vllm_plugin/tri_sample.py:275-290). Has no single-kernel counterpart in the reference, which
 * never shards the vocabulary. */
size_t bx_sample_scratch_bytes(int M, int V);
int bx_sample(const int64_t* logits, int64_t ld, const int64_t* rows, const int64_t* lnt, void* scratch,
              int64_t* tok, int M, int V, int bits, void* stream);
int bx_sample_shard(const int64_t* logits, int64_t ld, const int64_t* rows, const int64_t* lnt, void* scratch,
                    int64_t* best, int64_t* idx, int M, int V_local, int64_t v_offset, int bits, void* stream);

/* ---- weight preparation (load time) ----------------------------------------------------------------------------
 * bf16 weights w [N, K] (raw 16-bit patterns, row stride ldw) -> the constants of the exact-mode linear layer:
 * limbs int8 [3][N][K], per-row grid exponent g and residual depth d (int64 [N]), cnt int32 [N] = residual entries
 * of each row. flag (int32, OR-ed): 1 = inf / nan weight, 2 = residual grid finer than 30 bits, 4 = a value that
 * three limbs do not hold (the host code raises ValueError in these cases). Then, with start = the exclusive prefix
 * sum of cnt, bx_decompose_residual writes the coordinate list (rr, rc, rv int64 [sum cnt]) in row-major order.
 * Replaces exact.consts.decompose / bf16_parts (src/bitexact/exact/consts.py:33-107), which run on the host. */
int bx_decompose_rows(const uint16_t* w, int64_t ldw, int8_t* limbs, int64_t* g, int64_t* d, int32_t* cnt, int32_t* flag,
                      int N, int K, void* stream);
int bx_decompose_residual(const uint16_t* w, int64_t ldw, const int64_t* g, const int64_t* d, const int64_t* start,
                          int64_t* rr, int64_t* rc, int64_t* rv, int N, int K, void* stream);

/* ---- integer log p ---------------------------------------------------------------------------------------------
 * Integer log p of tok [M] under int64 logits rows [M, V] (row stride ld) at fr fractional bits (13..24; the
 * reference's int8 mode uses 16): out int64 [M] = the value at 2^-40; the caller converts to float64 as the
 * reference does. lnt = ln table int64 [65537] at 40 bits; tab = e^x at 44 bits for x in [-40, 0] at step 2^-12,
 * int64 [tab_len = 163841] (rl.lse_table, rl.py:32-40), handed over as tab2 = int64 [tab_len][2], 16-byte aligned,
 * tab2[i] = (tab[i], tab[min(i + 1, tab_len - 1)]) (bx_logp_pair_table builds it on the device, once per table);
 * scratch: bx_logp_scratch_bytes(M, V) bytes. A token outside [0, V) gives INT64_MIN in
 * its row (the reference's gather raises there). Replaces rl.int_logp (src/bitexact/vllm_plugin/rl.py:43-65) and
 * tri_logp.logp (src/bitexact/vllm_plugin/tri_logp.py:70-91). */
size_t bx_logp_scratch_bytes(int M, int V);
int bx_logp_pair_table(const int64_t* tab, int tab_len, int64_t* tab2, void* stream);
int bx_int_logp(const int64_t* logits, int64_t ld, const int64_t* tok, const int64_t* lnt, const int64_t* tab2,
                int tab_len, void* scratch, int64_t* out, int M, int V, int fr, void* stream);
/* The same computation in steps, for a COLUMN SHARD of the vocabulary: the shard's row maxima; the shard's sum of
 * e^(l - rowmax) terms against the maximum of the full row (the caller's all-reduce MAX of the shard maxima); and,
 * on [M], log p from the full sum S (the all-reduce SUM of the shard sums, < 2^62) and the target term
 * zt = l_tok - rowmax. Integer max and sum: every sharding gives the bits of the full row. The reference never
 * shards the vocabulary; its chunked kernels (_stat_kernel / _sum_kernel, tri_logp.py:27-67) are the same split
 * inside one GPU. */
int bx_logp_rowmax(const int64_t* logits, int64_t ld, void* scratch, int64_t* rowmax, int M, int V, void* stream);
int bx_logp_rowsum(const int64_t* logits, int64_t ld, const int64_t* rowmax, const int64_t* tab2, int tab_len,
                   void* scratch, int64_t* S, int M, int V, int fr, void* stream);
int bx_logp_finish(const int64_t* S, const int64_t* zt, const int64_t* lnt, int64_t* out, int M, int fr, void* stream);

#ifdef __cplusplus
}
#endif
#endif
