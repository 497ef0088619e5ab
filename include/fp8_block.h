/*
 * fp8_block.h — C ABI of libfp8block.so: the row-local glue of a Llama-style
 * decoder block fused with the per-tensor e4m3 quantiser that feeds the FP8 GEMM
 * and FP8 attention libraries, for NVIDIA B200 (sm_100a).
 *
 * What each entry point replaces in goml:
 *   - rmsnorm_forward / swiglu_forward / rope_forward of libtransformer.so
 *     (libs/transformer_kernels.cu:384-438), each followed at the call site by a
 *     separate quantiser launch (libs1/fp8_quantize_v2.cu:176-204) and, for the
 *     attention operands, by host round trips for amax and scale
 *     (internal/abjexam/battle_a_llm.go:380-494);
 *   - the [S,H,hd] <-> [H,S,hd] permutes of nn/attention.go:100-150.
 * The arithmetic is that of the reference's fp64 golden for the block
 * (internal/abjexam/llama_hf_f64ref.go:126-178, battle_a_llm_f64ref.go:182-194 and
 * :221-237): RMSNorm with eps inside the square root, half-split RoPE (pairs
 * (i, i + hd/2), angle = pos * theta^(-2i/hd)), SwiGLU silu(gate) * up — evaluated
 * in fp32 — followed by the quantiser of fp8_quantize.h with scale = amax / 448:
 *     amax  = max |y|,  scale = amax > 1e-12 ? amax / 448 : 1,  inv = 1 / scale,
 *     q     = e4m3_rn_satfinite(clamp(y * inv, -448, 448)).
 *
 * Every op is two passes over its input (the per-tensor amax must be known before
 * the first code is written): pass 1 reduces amax (and the row statistics), pass 2
 * recomputes the values and writes codes.  Nothing but the codes, one scale and one
 * amax per tensor (and, where stated, the updated residual stream) is written.
 *
 * All pointers are device pointers owned by the caller; calls are asynchronous on
 * `stream`, allocate nothing and clear the amax words themselves.  Activations that
 * come out of the FP8 GEMM are bf16, the attention output is fp16, the residual
 * stream is fp32.  Return value: cudaError_t as int, 0 = success;
 * cudaErrorInvalidValue for null/misaligned pointers or unsupported sizes.
 */
#ifndef GOML_FP8_BLOCK_H_
#define GOML_FP8_BLOCK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__) || defined(__clang__)
#define FP8BLOCK_API __attribute__((visibility("default")))
#else
#define FP8BLOCK_API
#endif

/* cos/sin tables for half-split RoPE: cos_out, sin_out [seq_len, head_dim/2] fp32,
 * angle = pos * theta^(-2i/head_dim) evaluated in fp64 (positions 0..seq_len-1). */
FP8BLOCK_API int fp8_rope_table(float* cos_out, float* sin_out, int seq_len, int head_dim, float theta, void* stream);

/* h = x (+ residual);  y = (h * gamma) * rsqrt(mean(h^2) + eps), each product rounded to fp32;  q = quantise(y).
 *   x [rows, hidden] fp32;  residual [rows, hidden] bf16 or NULL;
 *   h_out [rows, hidden] fp32 or NULL (may alias x): receives h when residual != NULL;
 *   gamma [hidden] fp32;  q [rows, hidden] e4m3;  rstd_ws [rows] fp32 scratch.
 * hidden must be a multiple of 16; x, h_out and gamma 32-byte aligned, the others 16-byte. */
FP8BLOCK_API int fp8_rmsnorm_quantize(const float* x, const void* residual_bf16, float* h_out, const float* gamma,
                                      uint8_t* q, float* scale_out, float* amax_out, float* rstd_ws, int rows,
                                      int hidden, float eps, void* stream);

/* qkv [batch*seq_len, 3, heads, head_dim] bf16 (the QKV projection's output rows)
 *   -> RoPE on Q and K -> q_out, k_out, v_out [batch*heads, seq_len, head_dim] e4m3,
 * each with its own per-tensor scale: scales[3], amaxes[3] (order Q, K, V).
 * head_dim 64 or 128. */
FP8BLOCK_API int fp8_rope_quantize_qkv(const void* qkv_bf16, const float* cos_tab, const float* sin_tab,
                                       uint8_t* q_out, uint8_t* k_out, uint8_t* v_out, float* scales, float* amaxes,
                                       int batch, int seq_len, int heads, int head_dim, void* stream);

/* Attention output o [batch*heads, seq_len, head_dim] fp16 -> token-major codes
 * q [batch*seq_len, heads*head_dim] e4m3 (the O projection's A operand).
 * head_dim a multiple of 16. */
FP8BLOCK_API int fp8_permute_quantize_heads(const void* o_fp16, uint8_t* q, float* scale_out, float* amax_out,
                                            int batch, int seq_len, int heads, int head_dim, void* stream);

/* gate_up [rows, 2*ffn_hidden] bf16 (gate columns first) -> silu(gate) * up ->
 * q [rows, ffn_hidden] e4m3.  ffn_hidden a multiple of 16; gate_up 32-byte aligned. */
FP8BLOCK_API int fp8_swiglu_quantize(const void* gate_up_bf16, uint8_t* q, float* scale_out, float* amax_out, int rows,
                                     int ffn_hidden, void* stream);

/* Single-pass quantiser for a bf16 tensor whose max|x| the producer already reduced into *amax_in (the SwiGLU
 * epilogue of fp8_gemm_swiglu does): scale = amax/448 as above, *scale_out written.  n a multiple of 16,
 * x 32-byte aligned. */
FP8BLOCK_API int fp8_quantize_bf16(const void* x_bf16, uint8_t* q, float* scale_out, const float* amax_in, size_t n,
                                   void* stream);

/* x[i] += y[i] (x fp32 residual stream, y bf16), n a multiple of 8. */
FP8BLOCK_API int fp8_residual_add(float* x, const void* y_bf16, size_t n, void* stream);

/* Decode step of quantised inference: the new token's projection row of every sequence -> RoPE at the token's
 * position -> Q codes for fa_decode, and the K and V codes appended to the FP8 KV cache in place.  It is the device
 * side of KVCache.Append(l, k, v) as sketched in runs/reports/F1_HF_INFERENCE_recon.md:186-196 (write position tCur
 * of a [H_kv, S_max, hd] cache), fused with RoPE (battle_a_llm_f64ref.go:221-237) and the quantiser.
 *   qkv_bf16   [batch, (q_heads + 2*kv_heads) * head_dim] bf16: query heads, then key heads, then value heads;
 *   cos_tab, sin_tab [rope_rows, head_dim/2] fp32 (fp8_rope_table);
 *   positions  [batch] int32 on the device: index of the new token = number of keys already cached.  A sequence whose
 *              position is outside [0, min(capacity, rope_rows)) is inactive: its Q codes are zeros, nothing is
 *              appended and its length is left as it is (seq_lens_out = 0 for a negative position, else
 *              min(position, capacity): a full cache stays full instead of wrapping around);
 *   q_out      [batch, q_heads, head_dim] e4m3 with a fresh per-tensor scale (*q_scale_out = amax/448, *q_amax_out);
 *   k_cache, v_cache: the layouts fa_decode reads -- [batch, kv_heads, s_max, head_dim], or with block_table != NULL
 *              pools [num_pages, kv_heads, page_size, head_dim] (block_table [batch, max_pages_per_seq] int32; a
 *              position whose table entry is outside [0, num_pages) is not written);
 *   k_scale, v_scale: device pointers to the dequantisation scales the cache was written with; the new codes are
 *              e4m3_rn_satfinite(clamp(x / scale)), i.e. values beyond 448 * scale saturate;
 *   seq_lens_out [batch] int32 or NULL: positions[b] + 1 for active sequences, the lengths to pass to fa_decode
 *              next (and the next step's positions); must not alias positions.
 * head_dim 64 or 128.  Two passes over the Q part (amax, then codes); K and V are written in the second. */
typedef struct fp8_decode_append_args {
    const void* qkv_bf16;
    const float* cos_tab;
    const float* sin_tab;
    const int32_t* positions;
    uint8_t* q_out;
    float* q_scale_out;
    float* q_amax_out;
    uint8_t* k_cache;
    uint8_t* v_cache;
    const float* k_scale;
    const float* v_scale;
    int32_t* seq_lens_out;
    const int32_t* block_table;
    int32_t batch, q_heads, kv_heads, head_dim;
    int32_t s_max, rope_rows;
    int32_t page_size, max_pages_per_seq, num_pages;
    int32_t reserved;
    void* stream;
} fp8_decode_append_args_t;

FP8BLOCK_API int fp8_decode_rope_append(const fp8_decode_append_args_t* args);

#ifdef __cplusplus
}
#endif
#endif
