/*
 * fp8_quantize.h — C ABI of libfp8quant.so: per-tensor FP32 -> FP8 (e4m3)
 * quantiser for NVIDIA B200 (sm_100a).
 *
 * Function and operation order follow goml's quantiser
 * (libs1/fp8_quantize_v2.cu:82-122 and :176-204):
 *     amax  = max |x|
 *     scale = amax > 1e-12 ? amax / DIV : 1          (IEEE fp32 division)
 *     inv   = 1 / scale                               (IEEE fp32 division)
 *     q     = e4m3_rn_satfinite(clamp(x * inv, -448, 448))
 * with DIV = 448 (the reference quantiser) or DIV = 1 ("unit" convention, decoded
 * magnitudes <= 1, the one goml's attention call site uses:
 * internal/abjexam/battle_a_llm.go:476-494).  The call shape — source, codes,
 * scale pointer, amax pointer, element count — is that call site's
 * QuantizeF32ToF8E4M3Unit(src, dst, scale, amax, n).
 *
 * All pointers are device pointers owned by the caller; the call is asynchronous
 * on `stream` and allocates nothing.  Unlike the reference call site the caller
 * does NOT have to zero `amax` first: the entry point clears it on `stream`
 * before reducing into it (the reference needed host syncs around a separate
 * zero-upload, battle_a_llm.go:463-473).
 * Return value: cudaError_t as int, 0 = success.
 */
#ifndef GOML_FP8_QUANTIZE_H_
#define GOML_FP8_QUANTIZE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__) || defined(__clang__)
#define FP8QUANT_API __attribute__((visibility("default")))
#else
#define FP8QUANT_API
#endif

#define FP8_QUANT_AMAX_OVER_448 0 /* scale = amax / 448 : codes span the e4m3 range */
#define FP8_QUANT_UNIT 1          /* scale = amax       : decoded magnitudes <= 1  */

/* Replaces the role of fp8_quantize_fp16 (libs1/fp8_quantize_v2.cu:176-204) for
 * FP32 sources.  x: n floats (16-byte aligned); q: n bytes (16-byte aligned);
 * scale_out, amax_out: one float each (both written). */
FP8QUANT_API int fp8_quantize_f32(const float* x, uint8_t* q, float* scale_out, float* amax_out, size_t n,
                                  int convention, void* stream);

/* Replaces fp8_dequantize_to_fp16 (libs1/fp8_quantize_v2.cu:206-214): out[i] =
 * fp16(decode(q[i]) * *scale_in). */
FP8QUANT_API int fp8_dequantize_to_fp16(const void* input_fp8, void* output_fp16, const float* scale_in, int n);

/* Replaces fp8_quantize_fp16 (libs1/fp8_quantize_v2.cu:176-204), same signature: n FP16 values -> n e4m3 codes with
 * scale = amax / 448 written to *scale_out; runs on the legacy default stream and returns without synchronising,
 * as the reference does.  Differences: argument errors return cudaErrorInvalidValue instead of faulting, and
 * nothing is allocated (the reference grows a cudaMalloc'ed reduction buffer; here the amax is one device word
 * inside the library, shared by all calls on a GPU, which the default stream serialises).  Codes and scale are
 * bit-identical to the reference's. */
FP8QUANT_API int fp8_quantize_fp16(const void* input_fp16, void* output_fp8, float* scale_out, int n);

/* Additive, no counterpart in the reference: the block-scaled ("MXFP8", OCP microscaling) quantiser that feeds
 * fp8_gemm_mx (libfp8gemm.so).  x is [rows, K] fp32 row-major, K a multiple of 128.  For every 32 consecutive elements
 * of a row: scale = 2^(floor(log2(amax)) - 8) (1 for an all-zero block), stored as ue8m0 (exponent + 127), and codes =
 * e4m3_rn_satfinite(x / scale) (values up to 2^9 occur before the conversion; those above 448 saturate, as the format
 * specifies).  q receives rows * K codes; scales receives ceil(rows / 128) * (K / 128) * 512 bytes in the tiled order
 * fp8_gemm_mx reads (include/fp8_gemm.h), padding entries set to scale 1.  x and q 16-byte aligned. */
FP8QUANT_API int fp8_quantize_mx_f32(const float* x, uint8_t* q, uint8_t* scales, int rows, int K, void* stream);

/* Replaces cuda_device_sync2 (libs1/fp8_quantize_v2.cu:216): cudaDeviceSynchronize() as int. */
FP8QUANT_API int cuda_device_sync2(void);

#ifdef __cplusplus
}
#endif
#endif
