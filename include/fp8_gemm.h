/*
 * fp8_gemm.h — C ABI of libfp8gemm.so, the FP8 (e4m3) GEMM
 *     C[M,N] = alpha * A[M,K] . B[N,K]^T          ("TN": both operands K-contiguous)
 * implemented for NVIDIA B200 (sm_100a) with tcgen05 tensor-core MMA.
 *
 * The first three entry points replace, symbol for symbol, the ones goml binds
 * with purego in backend/cuda/fp8_gemm.go:27-62 and that its libs/fp8_gemm.cu:315-353
 * defines.  Conventions kept from there:
 *   - every pointer is a device pointer owned by the caller; nothing is allocated
 *     or freed; the call is asynchronous on `stream` (NULL = default stream) and
 *     never synchronises the host;
 *   - the return value is a cudaError_t as int, 0 = success;
 *   - A is [M,K] row-major u8 (e4m3 codes), B is [N,K] row-major u8 (i.e. the
 *     [out,in] weight layout of nn/linear.go:14), C is [M,N] row-major;
 *   - K must be a multiple of 16 and A, B 16-byte aligned (libs/fp8_gemm.cu:83-103
 *     loads 16-byte units); violations return cudaErrorInvalidValue (1) here
 *     instead of reading out of bounds;
 *   - the calling thread's current device is used; per-device state is kept
 *     per device and the current device is never changed.
 * Deliberate differences: accumulation is FP32 in tensor memory (the reference
 * accumulates in FP16 and overflows above 65504); an odd N is handled (the
 * reference drops the last column, libs/fp8_gemm.cu:122-125).
 */
#ifndef GOML_FP8_GEMM_H_
#define GOML_FP8_GEMM_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__) || defined(__clang__)
#define FP8GEMM_API __attribute__((visibility("default")))
#else
#define FP8GEMM_API
#endif

/* Replaces fp8_gemm of libs/fp8_gemm.cu:315-340.  C is FP16, alpha = 1.
 * mode: 0 or 1 (the reference's "original"/"singlesync" kernels); any other
 * value is treated as 1.  Both modes run the same sm_100a kernel. */
FP8GEMM_API int fp8_gemm(int M, int N, int K, const void* A, const void* B, void* C, int mode, void* stream);

/* Replaces fp8_gemm_original of libs/fp8_gemm.cu:343-347. */
FP8GEMM_API int fp8_gemm_original(int M, int N, int K, const void* A, const void* B, void* C, void* stream);

/* Replaces fp8_gemm_singlesync of libs/fp8_gemm.cu:349-353. */
FP8GEMM_API int fp8_gemm_singlesync(int M, int N, int K, const void* A, const void* B, void* C, void* stream);

/* Additive extension (no counterpart in the reference ABI, which cannot express
 * per-tensor dequantisation or a BF16 result):
 *   C = (alpha * (*scale_a) * (*scale_b)) * A . B^T
 * scale_a / scale_b are optional DEVICE pointers to one float each (the scales a
 * quantiser wrote; NULL = 1), read by the kernel so no host round trip is needed.
 * out_dtype: 0 = FP16, 1 = BF16. */
#define FP8_GEMM_OUT_FP16 0
#define FP8_GEMM_OUT_BF16 1
FP8GEMM_API int fp8_gemm_scaled(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                                const float* scale_a, const float* scale_b, int out_dtype, void* stream);

/* Additive extension: the residual-stream update of a decoder block in the GEMM epilogue,
 *   X[M,N] (fp32, row-major) += (alpha * (*scale_a) * (*scale_b)) * A . B^T
 * read-modify-write with 128-bit accesses; takes the place of a 16-bit result followed by
 * a separate add pass over X (x = x + W y in internal/abjexam/llama_hf_f64ref.go:150,178).
 * The fp32 accumulators are added un-rounded.  A problem with few output tiles and a long K (M <= 128 rows against a
 * wide weight) is divided over K among several thread blocks, each adding its partial sum into X: the result is then
 * the same sum in an order that is not fixed from run to run (differences in the last bits of fp32). */
FP8GEMM_API int fp8_gemm_accumulate_f32(int M, int N, int K, const void* A, const void* B, float* X, float alpha,
                                        const float* scale_a, const float* scale_b, void* stream);

/* Additive extension: the SwiGLU feed-forward's gate and up projections with the activation in the epilogue,
 *   H[M,F] (bf16) = silu(g) * u,   g = s * A . Wgate^T,   u = s * A . Wup^T,   s = alpha * (*scale_a) * (*scale_b)
 * (silu(x) = x / (1 + e^-x); nn/feedforward.go:54-79 computes W2(silu(W1 x) * W3 x)), and max|H| reduced into
 * *amax_out (cleared by the call) for the per-tensor quantiser of the down projection's operand.
 * B_interleaved holds both weights, [2 * Fp, K] with Fp = F rounded up to 32: rows [64t, 64t+32) are rows
 * [32t, 32t+32) of Wgate, rows [64t+32, 64t+64) the same rows of Wup; rows past F are zero (every tile width the
 * kernel uses, 64 to 256 columns, then holds whole gate/up pairs, so small M runs on narrow tiles).
 * The 16-bit gate/up matrix is never written. */
FP8GEMM_API int fp8_gemm_swiglu(int M, int F, int K, const void* A, const void* B_interleaved, void* H, float alpha,
                                const float* scale_a, const float* scale_b, float* amax_out, void* stream);

/* Additive extension: e4m3 output with delayed scaling, the epilogue of the reference's cuBLASLt wrapper
 * (fp8_matmul_fp8out, libs1/cublas_lt_wrapper_v3.c:157-229: D type CUDA_R_8F_E4M3 with D_SCALE_POINTER and
 * AMAX_D_POINTER):
 *   v = s * A . B^T,  s = alpha * (*scale_a) * (*scale_b), rounded to fp32;
 *   D[M,N] (e4m3, row-major) = e4m3_rn_satfinite((*scale_d) * v);   *amax_d = max |v|  (before scale_d).
 * scale_d is the MULTIPLIER applied before the conversion (the consumer dequantises with 1 / *scale_d); NULL = 1.
 * amax_d may be NULL; otherwise the call clears it and the kernel reduces into it, so the caller can derive the
 * next call's scale_d from it.  D must be 16-byte aligned and N a multiple of 16 for vector stores; other shapes
 * take a byte-store path. */
FP8GEMM_API int fp8_gemm_fp8out(int M, int N, int K, const void* A, const void* B, void* D, float alpha,
                                const float* scale_a, const float* scale_b, const float* scale_d, float* amax_d,
                                void* stream);

/* Additive, no counterpart in the reference (its roadmap's next step, docs/FP8_FA_ROADMAP.md:137-148): the block-scaled
 * ("MXFP8") GEMM.  A and B are e4m3 codes as before; every row of A and of B carries one ue8m0 scale (a power of two,
 * byte = exponent + 127, 0xFF is NaN) per 32 consecutive K elements, and
 *   C[m,n] = alpha * sum over K blocks kb of 2^(ea[m,kb] + eb[n,kb]) * (A[m, 32 kb .. 32 kb + 31] . B[n, 32 kb .. 32 kb + 31]),
 * the scales applied inside the tensor-core instruction (tcgen05.mma kind::mxf8f6f4.block_scale), fp32 accumulation,
 * FP16 or BF16 output.  K must be a multiple of 128.
 * Scale arrays (scale_a for the M rows of A, scale_b for the N rows of B) are device arrays of fp8_mx_scale_bytes(rows, K)
 * bytes in the order the kernel copies them: for row tile rt = row / 128 and slab ks = kb / 4 the 512 bytes at
 * (rt * (K / 128) + ks) * 512 hold, at byte ((row % 32) * 16 + ((row % 128) / 32) * 4 + kb % 4), the scale of (row, kb);
 * entries of rows past the matrix must not be 0xFF.  fp8_quantize_mx_f32 (libfp8quant.so) writes codes and scales in
 * this form.  A, B, scale_a, scale_b 16-byte aligned. */
FP8GEMM_API size_t fp8_mx_scale_bytes(int rows, int K);
FP8GEMM_API int fp8_gemm_mx(int M, int N, int K, const void* A, const void* scale_a, const void* B, const void* scale_b, void* C,
                            float alpha, int out_dtype, void* stream);
/* Bounded-wait status of the block-scaled kernel (as fp8_gemm_device_status). */
FP8GEMM_API int fp8_gemm_mx_device_status(void);

/* Additive: tile-pair policy of this process.  mode -1 = chosen per problem (default), 0 = large problems run as
 * single 128 x 256 tiles instead of 256-row tile pairs; other values return cudaErrorInvalidValue.  Results are
 * bit-identical either way (a switch for comparisons, not needed in production).  The environment variable
 * FP8_GEMM_NO_PAIR (any value) selects mode 0; it is read once, at the first launch of the process, and a call of
 * this function overrides it. */
FP8GEMM_API int fp8_gemm_set_tile_pairs(int mode);

/* Additive: device-side status of the current device.  The kernels bound every
 * wait; if a wait ever runs out they record a non-zero code here and exit
 * cleanly.  This call synchronises the device and returns (and clears) the
 * code; 0 = no kernel reported a problem.  Negative = CUDA error code negated. */
FP8GEMM_API int fp8_gemm_device_status(void);

/* Additive: self-test of the bounded waits.  Launches one warp that waits, with a 1 ms budget, on a barrier nothing
 * ever arrives at; the wait gives up and the kernel returns after latching code 0x1F0 the way a production kernel's
 * teardown would.  The next fp8_gemm_device_status() must therefore return 0x1F0, and the one after that 0.  Touches
 * no operand memory, no TMA, no tensor memory; the GPU context stays usable. */
FP8GEMM_API int fp8_gemm_selftest_wait_expiry(void* stream);

/* Additive: static version string. */
FP8GEMM_API const char* fp8_gemm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GOML_FP8_GEMM_H_ */
