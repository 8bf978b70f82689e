/*
 * dgq.h - C ABI of the B200 (sm_100a) GPTQ quantization path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes, is
 * asynchronous on the CUDA stream it is given (a `cudaStream_t` passed as
 * `void*`; NULL is the default stream) and returns a status: 0 = enqueued,
 * negative = rejected on the host before any launch (see DGQ_ERR_*).
 * The library never allocates or frees device memory: the caller owns every
 * buffer, including the workspaces sized by the *_workspace_bytes functions.
 * Conditions found on the device (a non-positive Cholesky pivot, a bounded wait
 * that ran out) are written to the caller's `info` words, which the caller reads
 * after synchronising.
 *
 * Each declaration names the reference interface it stands in for, as
 * file:line inside the reference project (src/distributed_gptq/...).
 *
 * Matrices are row-major.  W is (N_out, K): rows are output features, columns
 * are input features, so columns line up with the K x K Hessian.
 */
#ifndef DGQ_H_
#define DGQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define DGQ_OK                 0
#define DGQ_ERR_ARG          (-1)  /* null pointer, non-positive size, unknown enum */
#define DGQ_ERR_ALIGN        (-2)  /* pointer or leading dimension not aligned as documented */
#define DGQ_ERR_WORKSPACE    (-3)  /* workspace smaller than *_workspace_bytes() */
#define DGQ_ERR_ARCH         (-4)  /* current device is not compute capability 10.x */
#define DGQ_ERR_LAUNCH       (-5)  /* the CUDA runtime refused a launch or a set-up call */
#define DGQ_ERR_UNSUPPORTED  (-6)  /* valid request outside what this build implements */
#define DGQ_ERR_SIZE         (-7)  /* size beyond a documented maximum */

/* device-side conditions, written to info[0] (info[1] holds a detail word) */
#define DGQ_INFO_OK              0
#define DGQ_INFO_NOT_POSDEF      1  /* info[1] = index of the first non-positive pivot */
#define DGQ_INFO_WAIT_TIMEOUT    2  /* info[1] = which wait gave up */

/* ---- enums -------------------------------------------------------------- */
/* packing formats */
#define DGQ_FMT_BYTES_HI_FIRST   1  /* GPTQ.pack_weights, core/gptq.py:229-257 */
#define DGQ_FMT_BYTES_LO_FIRST   2  /* QuantizedLinear.pack_weights, models/layers.py:76-93 */
#define DGQ_FMT_INT32_LE         3  /* pack_weights_kernel, kernels/triton_kernels.py:203-222 */
/* element types of float buffers */
#define DGQ_F32   0
#define DGQ_F16   1
#define DGQ_BF16  2

const char* dgq_status_string(int32_t status);
int32_t     dgq_version(void);
/* 0 when the current device can run this library (compute capability 10.x). */
int32_t     dgq_device_check(void);
/* Number of CUDA kernels this library has launched in this process so far.  It has
 * no counterpart in the reference; the benchmark reports it as evidence that the
 * timed work ran in these kernels. */
int64_t     dgq_launch_count(void);

/* ---- Hessian accumulation ------------------------------------------------
 * Replaces GPTQ.add_batch, core/gptq.py:63-89 (`self.H += inp @ inp.t()`).
 *
 * H(K,K) += alpha * X^T X with X (T,K) bf16 row-major, fp32 accumulation on the
 * 5th-generation tensor cores (TMA -> shared memory -> tcgen05.mma -> TMEM).
 * The full symmetric matrix is updated.  Requirements: X 16-byte aligned,
 * ldx (elements) a multiple of 8, K >= 8, H 16-byte aligned, ldh a multiple of 4.
 * `info` (device, 2 x int32, or NULL) receives DGQ_INFO_WAIT_TIMEOUT if a bounded
 * wait inside the kernel ran out; it is never cleared by the library.
 * `splits` >= 1 fixes the number of token ranges the work is cut into (each
 * range adds into H with fp32 reductions, so splits > 1 is not bit-reproducible);
 * 0 lets the library choose.
 */
int32_t dgq_hessian_accum(const void* X_bf16, int64_t T, int32_t K, int64_t ldx,
                          float* H, int64_t ldh, float alpha, int32_t splits,
                          int32_t* info, void* stream);

/* The same accumulation restricted to the part of H on and above the diagonal; what lies
 * below the diagonal is neither read nor written.  X^T X is symmetric, so a caller that
 * accumulates many batches (core/gptq.py:63-89 is called once per calibration batch) can
 * skip the mirrored half of every update - half of the kernel's reduction traffic - and call
 * dgq_hessian_mirror once, before the matrix is read as a whole (core/gptq.py:112-122).
 * H is only ever the target of fp32 reductions (nothing is loaded from it), so it may be the
 * memory of another GPU mapped into this process: ranks that all pass the buffer of the rank
 * that will quantize the layer have summed their partial Hessians (the all_reduce of
 * distributed/coordinator.py:224) when their launches have completed.
 */
int32_t dgq_hessian_accum_upper(const void* X_bf16, int64_t T, int32_t K, int64_t ldx,
                                float* H, int64_t ldh, float alpha, int32_t splits,
                                int32_t* info, void* stream);
/* H[i][j] = H[j][i] for i > j. */
int32_t dgq_hessian_mirror(float* H, int32_t K, int64_t ldh, void* stream);

/* fp32 -> bf16 (round to nearest even) for activations that arrive as fp32
 * (core/gptq.py:88 upcasts; the tensor-core path takes bf16). n elements. */
int32_t dgq_cast_f32_to_bf16(const float* src, void* dst_bf16, int64_t n, void* stream);
/* fp16 -> bf16 */
int32_t dgq_cast_f16_to_bf16(const void* src_f16, void* dst_bf16, int64_t n, void* stream);

/* ---- Hessian preparation --------------------------------------------------
 * Replaces core/gptq.py:112-119 (normalise + damp) and adds what the reference
 * stores but never applies (act-order, core/gptq.py:49) and dead-column handling.
 *
 * dgq_actorder_perm: perm = stable argsort, in descending order (ties keep
 *   ascending index), of the prepared diagonal scale*H_ii with zero entries read
 *   as 1; invperm[perm[i]] = i.
 * dgq_hessian_prepare: Hout[i][j] = scale * H[p(i)][p(j)]  (p = perm, or identity
 *   when perm is NULL); a zero diagonal entry becomes 1 and marks the column dead;
 *   then diag += percdamp * mean(diag).  dead_out (K bytes, in permuted order)
 *   receives the dead mask.  H and Hout must not overlap.  ws: 256 bytes.
 * dgq_permute_cols_f32: dst[r][i] = dead && dead[i] ? 0 : src[r][perm[i]]
 * dgq_permute_cols_u8 : dst[r][i] = src[r][perm[i]]
 * dgq_permute_cols_u16: the same for 16-bit elements (fp16 / bf16 activations brought into the
 *   column order of an act-order layer before the quantized linear, models/layers.py:150-153)
 */
int32_t dgq_actorder_perm(const float* H, int32_t K, int64_t ldh, float scale,
                          int32_t* perm, int32_t* invperm, void* stream);
int64_t dgq_hessian_prepare_workspace_bytes(int32_t K);
int32_t dgq_hessian_prepare(const float* H, int64_t ldh, float* Hout, int64_t ldo, int32_t K,
                            float scale, float percdamp, const int32_t* perm,
                            uint8_t* dead_out, void* ws, int64_t ws_bytes, void* stream);
int32_t dgq_permute_cols_f32(const float* src, int64_t lds, float* dst, int64_t ldd,
                             int32_t rows, int32_t cols, const int32_t* perm,
                             const uint8_t* dead, void* stream);
int32_t dgq_permute_cols_u8(const uint8_t* src, int64_t lds, uint8_t* dst, int64_t ldd,
                            int32_t rows, int32_t cols, const int32_t* perm, void* stream);
int32_t dgq_permute_cols_u16(const void* src, int64_t lds, void* dst, int64_t ldd,
                             int32_t rows, int32_t cols, const int32_t* perm, void* stream);

/* ---- damped inverse -------------------------------------------------------
 * Replaces core/gptq.py:121-122 (`cholesky_inverse(linalg.cholesky(H))`) and the
 * upper-Cholesky step of the GPTQ algorithm.
 *
 * In place: A (K,K) symmetric positive definite (only its upper triangle and
 * diagonal are read) -> U upper triangular with A^-1 = U^T U; the strict lower
 * triangle of the result is zero.  Recursive blocked fp32 factorisation on the device
 * (fp32-accurate tensor-core products above 128 x 128, one CTA per 128 x 128 leaf).
 * info (device, 2 x int32): DGQ_INFO_NOT_POSDEF and the pivot index on failure.
 * lda a multiple of 4, A 16-byte aligned.
 * Part of the work runs on a side stream that the library creates on first use for
 * every (host thread, device, caller stream) and joins back into `stream` before the
 * call's last kernels, so the call is ordered on `stream` like any other.  Make the
 * first call for a stream outside a stream capture (streams and events are created).
 */
int64_t dgq_inv_chol_workspace_bytes(int32_t K);
int32_t dgq_inv_chol_upper(float* A, int32_t K, int64_t lda, int32_t* info,
                           void* ws, int64_t ws_bytes, void* stream);

/* ---- fp32-accurate matrix product on the tensor cores -------------------------
 * The product behind the inverse factor and the trailing update
 * (`W_block[:, j+1:] -= err @ H_inv[j, j+1:]` batched over a block, core/gptq.py:187,
 * and the products inside torch.cholesky_inverse, core/gptq.py:122), exported so that it
 * can be checked on its own.
 *
 * C(m,n) = alpha * A(m,k) * B + beta * C, all fp32 row-major.  B is (n,k) when
 * b_is_kn == 0 (C = A * B^T) and (k,n) otherwise.  Operands are split into tf32 high
 * and low parts and three tcgen05 products are accumulated, so results agree with an
 * fp32 product to about 1e-6 relative.  lower_only != 0 computes and writes only
 * entries with column <= row.  Bases 16-byte aligned, leading dimensions multiples of 4.
 */
int32_t dgq_gemm_f32(const float* a, int64_t lda, const float* b, int64_t ldb, int32_t b_is_kn,
                     float* c, int64_t ldc, int32_t m, int32_t n, int32_t k,
                     float alpha, float beta, int32_t lower_only, int32_t* info, void* stream);

/* ---- blockwise quantization -----------------------------------------------
 * Replaces the block/column loop of GPTQ.quantize, core/gptq.py:131-194, with the
 * scale/zero formula of :165-169 and the quantize/dequantize formula of :175,179.
 *
 * W (N_out,K) fp32 in/out: on return it holds the dequantized weights Q.
 * U (K,K): the factor from dgq_inv_chol_upper.  codes (N_out,K) uint8.
 * scales/zeros (N_out, n_groups) fp32 with n_groups = ceil(K/group_size), or 1 when
 * group_size <= 0 or >= K (per output channel).  total_error: one device double,
 * receives sum(((w - w_hat)/d)^2) (core/gptq.py:183,191); it is overwritten.
 * blocksize must be 128 or less and group_size, when it is smaller than K, must
 * either divide blocksize or be a multiple of it.  The workspace holds scaled errors:
 * dgq_gptq_quantize_workspace_bytes() asks for N_out x 256 floats (updates of far columns
 * are then batched over 256 columns); any size down to N_out x 128 floats is accepted.
 */
int64_t dgq_gptq_quantize_workspace_bytes(int32_t N_out, int32_t K, int32_t blocksize);
int32_t dgq_gptq_quantize(float* W, int64_t ldw, const float* U, int64_t ldu,
                          int32_t N_out, int32_t K, int32_t bits, int32_t group_size,
                          int32_t blocksize, uint8_t* codes, int64_t ldc,
                          float* scales, float* zeros, double* total_error,
                          void* ws, int64_t ws_bytes, void* stream);

/* dgq_gptq_quantize with one more output: row_error (N_out doubles, may be null) receives
 * sum(((w - w_hat)/d)^2) of every weight row, the per-row split of total_error
 * (core/gptq.py:183,191).  Rows are independent given U, so layers that read the same
 * input (one Hessian, one U: q/k/v or gate/up of a decoder block) can be quantized as one
 * stacked matrix; the per-layer `total_error` of the reference's stats (core/gptq.py:203-210)
 * is then the sum of the layer's rows.
 */
int32_t dgq_gptq_quantize_rows(float* W, int64_t ldw, const float* U, int64_t ldu,
                               int32_t N_out, int32_t K, int32_t bits, int32_t group_size,
                               int32_t blocksize, uint8_t* codes, int64_t ldc,
                               float* scales, float* zeros, double* total_error,
                               double* row_error, void* ws, int64_t ws_bytes, void* stream);

/* Same computation as dgq_gptq_quantize for callers that must not allocate device
 * memory - code running inside another framework's memory plan, or under an allocator
 * that forbids cudaMalloc while a model is resident - and so cannot provide the
 * workspace.  It has no counterpart in the reference.  The scaled-error scratch lives in a
 * fixed array inside the library's device image (8 MiB per GPU that loads the library,
 * held until the process exits), which limits N_out to
 * dgq_gptq_quantize_noalloc_max_rows() = 16384 rows; more rows are rejected with
 * DGQ_ERR_SIZE.  The call makes no cudaMalloc/cudaFree and uses no allocating library
 * routine.  The first call on a device looks up the array's device address (a host-side
 * set-up step): make that first call before starting any stream capture.  All calls on
 * a device share the one array, whose contents are whatever the last call left (every
 * entry that is read is written first, so nothing needs clearing); two calls that
 * overlap on the same GPU - different streams or threads - race on it and must be
 * serialised by the caller.
 */
int32_t dgq_gptq_quantize_noalloc_max_rows(void);
int32_t dgq_gptq_quantize_noalloc(float* W, int64_t ldw, const float* U, int64_t ldu,
                                  int32_t N_out, int32_t K, int32_t bits, int32_t group_size,
                                  int32_t blocksize, uint8_t* codes, int64_t ldc,
                                  float* scales, float* zeros, double* total_error,
                                  void* stream);

/* ---- scale/zero and quantize on their own ("Quantizer.find_params/quantize") --
 * find_params: per row of x (rows, cols): scale = (max-min)/maxq (1 if zero),
 *   zero = round(-min/scale)                       (core/gptq.py:165-169)
 * quantize_rows: q = clamp(round(x/scale + zero), 0, maxq), x_hat = (q-zero)*scale
 *   with one (scale, zero) per row; either output may be NULL. (core/gptq.py:175,179)
 */
int32_t dgq_find_params(const float* x, int64_t ldx, int32_t rows, int32_t cols, int32_t bits,
                        float* scale, float* zero, void* stream);
int32_t dgq_quantize_rows(const float* x, int64_t ldx, int32_t rows, int32_t cols, int32_t bits,
                          const float* scale, const float* zero,
                          uint8_t* q, int64_t ldq, float* x_hat, int64_t ldh, void* stream);

/* ---- packing and dequantization -------------------------------------------
 * dgq_pack replaces GPTQ.pack_weights (core/gptq.py:229-257, format 1),
 * QuantizedLinear.pack_weights (models/layers.py:76-93, format 2) and
 * pack_weights_kernel (kernels/triton_kernels.py:203-222, format 3).
 * codes (rows, cols) uint8, contiguous.  Packed row length in bytes:
 *   format 1: cols*bits/8 for 2- and 4-bit (cols must divide evenly), cols otherwise;
 *   format 2: ceil(cols/2) for 4-bit, cols otherwise;
 *   format 3: 4*ceil(cols / (32/bits)).
 * dgq_packed_row_bytes returns that length (negative status on bad arguments).
 * dgq_unpack is the inverse (QuantizedLinear.unpack_weights models/layers.py:105-120,
 * GPTQDequantizer._unpack_4bit core/dequantizer.py:68-89).
 * dgq_unpack_dequant fuses the inverse with (code - zero[r][g]) * scale[r][g]
 * (models/layers.py:122-136, core/dequantizer.py:31-66, dequantize_kernel
 * kernels/triton_kernels.py:82-123); g = g_idx[c] when g_idx is given, else
 * c / group_size (one group when group_size <= 0 or >= cols).  scales/zeros are
 * (rows, n_groups) of param_dtype (DGQ_F32 or DGQ_F16); out is (rows, cols) of
 * out_dtype, contiguous.
 */
int64_t dgq_packed_row_bytes(int32_t cols, int32_t bits, int32_t format);
int32_t dgq_pack(const uint8_t* codes, int32_t rows, int32_t cols, int32_t bits, int32_t format,
                 void* packed, void* stream);
int32_t dgq_unpack(const void* packed, int32_t rows, int32_t cols, int32_t bits, int32_t format,
                   uint8_t* codes, void* stream);
int32_t dgq_unpack_dequant(const void* packed, const void* scales, const void* zeros,
                           const int32_t* g_idx, int32_t rows, int32_t cols, int32_t n_groups,
                           int32_t bits, int32_t group_size, int32_t format,
                           int32_t param_dtype, int32_t out_dtype, void* out, void* stream);

/* ---- quantized linear -------------------------------------------------------
 * Implements the operator QuantizedLinear.forward dispatches to,
 * torch.ops.gptq.linear(x, qweight, scales, zeros, g_idx, bias)
 * (models/layers.py:150-153), and stands in for quantized_matmul_kernel
 * (kernels/triton_kernels.py:126-183).
 *
 * y(M,N_out) = x(M,K) * dequant(qweight)^T + bias, fp32 accumulation.
 * qweight is in the QuantizedLinear layout (format 2: nibble pairs for 4-bit, one
 * byte per code otherwise); scales/zeros (N_out, n_groups) fp16; g_idx (K) int32
 * group of every input column, or NULL for c / group_size; bias (N_out) of
 * bias_dtype or NULL; x and y of x_dtype (DGQ_F32, DGQ_F16 or DGQ_BF16).
 * Up to 32 rows the call is bound by the packed weights' HBM traffic and runs in chunks of 16
 * rows on kernels that read every weight byte once.  From 33 rows on (prefill-sized M;
 * 4-bit codes, 16-bit activations, no g_idx, K and the group size multiples of 64) one
 * tcgen05 kernel does the whole product: weights are dequantized into shared memory as the
 * second operand, activations arrive by TMA, fp32 accumulation in tensor memory - the
 * 128 x 128 x K tiling kernels/triton_kernels.py:126-183 sketches.
 */
int32_t dgq_qlinear_forward(const void* x, int32_t x_dtype, int32_t M,
                            const uint8_t* qweight, const void* scales_f16, const void* zeros_f16,
                            const int32_t* g_idx, const void* bias, int32_t bias_dtype,
                            int32_t N_out, int32_t K, int32_t n_groups, int32_t bits,
                            int32_t group_size, void* y, void* stream);

/* ---- flat round-to-nearest helpers ------------------------------------------
 * Replace quantize_kernel / dequantize_kernel and the host loops around them
 * (kernels/triton_kernels.py:34-123, 377-481).  Groups are runs of group_size
 * consecutive elements of the flattened tensor; scale = (max-min)/maxq (1 if
 * zero), zero = -min/scale (not rounded, :411).
 */
int32_t dgq_rtn_find_params(const float* x, int64_t n, int32_t bits, int32_t group_size,
                            float* scales, float* zeros, void* stream);
int32_t dgq_rtn_quantize(const float* x, int64_t n, int32_t bits, int32_t group_size,
                         const float* scales, const float* zeros, uint8_t* q, void* stream);
int32_t dgq_rtn_dequantize(const uint8_t* q, int64_t n, int32_t group_size,
                           const float* scales, const float* zeros, float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DGQ_H_ */
