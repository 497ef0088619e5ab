/*
 * fa_sm120.h — C ABI of libfa_sm120.so as built for NVIDIA B200 (sm_100a):
 * FP8 (e4m3) FlashAttention forward, head_dim 64 and 128, causal and
 * sliding-window masks, optional log-sum-exp output.
 *
 * The library keeps the file name and the nine entry points of goml's
 * libs/fa_sm120/include/fa_sm120.h:66-150, so that its loaders
 * (backend/cuda/fa_forward.go:74-183 via purego, libs/fa_sm120/go/gofa/gofa.go via
 * cgo, libs/fa_sm120/python/fa_sm120.py via ctypes) bind it unchanged.  Each
 * declaration below cites the reference declaration it replaces.
 *
 * Conventions (as in the reference): C linkage, opaque context, status codes,
 * no exceptions and no printing; all tensors are device memory owned by the
 * caller, tightly packed [batch_heads, seq_len, head_dim] row-major; Q, K, V are
 * e4m3 bytes, O is fp16, the LSE is fp32 [batch_heads, seq_len]; calls are
 * asynchronous on `stream`; one context serves one GPU (the device current at
 * fa_create) and distinct contexts may be used from distinct threads.
 *
 * What differs from the sm_120a build, deliberately:
 *   - fa_create accepts compute capability 10.x and rejects everything else;
 *   - every (head_dim, mask, window) cell runs, through both fa_forward and
 *     fa_forward_train (the reference launches only its hd128 "v121r" cell and
 *     returns FA_ERR_INTERNAL for the rest, src/fa_ctx.cu:146-172, and its
 *     train entry is hd128 only, src/fa_ctx.cu:214-217);
 *   - accumulation is fp32 (the reference accumulates in fp16 and therefore
 *     needs decoded |Q|,|K|,|V| = O(1), fa_sm120.h:15-25); both "scale = amax"
 *     and "scale = amax/448" quantisation are fine here;
 *   - keys at or beyond seq_len are masked for every mask mode (the reference
 *     masks them only when causal = 1, src/_v121r_train_kernel.cu:468-496);
 *   - Q, K, V and O must be 16-byte aligned (FA_ERR_INVALID_ARG otherwise).
 */
#ifndef FA_SM120_H_
#define FA_SM120_H_

#ifdef __cplusplus
extern "C" {
#endif

#include <stdint.h>

#if defined(__GNUC__) || defined(__clang__)
#define FA_API __attribute__((visibility("default")))
#else
#define FA_API
#endif

/* replaces fa_sm120.h:45 */
typedef struct fa_ctx fa_ctx_t;

/* replaces fa_sm120.h:47-56 (same values) */
typedef enum {
    FA_OK = 0,
    FA_ERR_INVALID_ARG = 1,
    FA_ERR_UNSUPPORTED_ARCH = 2,  /* GPU is not compute capability 10.x */
    FA_ERR_UNSUPPORTED_HD = 3,    /* head_dim not in {64, 128} */
    FA_ERR_UNSUPPORTED_SHAPE = 4,
    FA_ERR_CUDA = 5,              /* CUDA runtime error, text in fa_last_cuda_error */
    FA_ERR_OOM = 6,
    FA_ERR_INTERNAL = 7
} fa_status_t;

/* replaces fa_sm120.h:59 */
typedef struct CUstream_st* fa_stream_t;

/* replaces fa_create, fa_sm120.h:66.  Probes the current device.  On a device
 * that is not compute capability 10.x it returns FA_ERR_UNSUPPORTED_ARCH and,
 * like the reference (src/fa_ctx.cu:75-82), still hands back a context whose
 * fa_last_cuda_error explains why; the caller destroys it. */
FA_API fa_status_t fa_create(fa_ctx_t** ctx_out);

/* replaces fa_forward, fa_sm120.h:86-91.
 *   scale  = softmax_scale * scale_Q * scale_K (one float applied to Q.K^T)
 *   causal in {0,1}; window in [0, seq_len], 0 = none.
 *   causal=1, window=w: query i sees keys [max(0, i-w+1), i].
 *   causal=0, window=w: query i sees keys [max(0, i-w+1), seq_len)  — the meaning
 *   the reference's CPU check gives it
 *   (libs/flash_attention_v121r_diet_hd128_fp8_forward.cu:721-724).
 * O is in decoded-V units (multiply by scale_V afterwards, as
 * internal/abjexam/battle_a_llm.go:534-544 does) — or use fa_forward_ex. */
FA_API fa_status_t fa_forward(fa_ctx_t* ctx, const void* q, const void* k, const void* v, void* o,
                              int batch_heads, int seq_len, int head_dim, int causal, int window,
                              float scale, fa_stream_t stream);

/* replaces fa_forward_train, fa_sm120.h:110-115.  As fa_forward plus
 * l_out[bh, sl] = natural-log LSE of the scaled scores (fa_sm120.h:100-102);
 * l_out may be NULL.  A row with no visible key gets O = 0 and LSE = -inf. */
FA_API fa_status_t fa_forward_train(fa_ctx_t* ctx, const void* q, const void* k, const void* v, void* o,
                                    void* l_out, int batch_heads, int seq_len, int head_dim, int causal,
                                    int window, float scale, fa_stream_t stream);

/* replaces fa_destroy, fa_sm120.h:120 (FA_OK on NULL) */
FA_API fa_status_t fa_destroy(fa_ctx_t* ctx);

/* replace fa_version / fa_status_str / fa_last_cuda_error, fa_sm120.h:125-127.
 * fa_last_cuda_error returns text owned by the context ("" for NULL). */
FA_API const char* fa_version(void);
FA_API const char* fa_status_str(fa_status_t);
FA_API const char* fa_last_cuda_error(fa_ctx_t* ctx);

/* replaces fa_kernel_id_t, fa_sm120.h:133-145.  On sm_100a one kernel family
 * serves every cell; the ids are kept as tile-configuration labels so that the
 * reference's dispatcher table test (libs/fa_sm120/test/test_dispatch.c) and
 * libs/fa_sm120/go/gofa/gofa_test.go:15-37 hold unchanged. */
typedef enum {
    FA_KERNEL_NONE = -1,
    FA_KERNEL_V121R = 100,
    FA_KERNEL_V121 = 101,
    FA_KERNEL_V118 = 102,
    FA_KERNEL_V122 = 103,
    FA_KERNEL_V117B = 104,
    FA_KERNEL_V96B = 105,
    FA_KERNEL_V89 = 200,
    FA_KERNEL_V80B = 201
} fa_kernel_id_t;

/* replaces fa_dispatch_select, fa_sm120.h:147-148 (pure function, same table as
 * src/fa_dispatch.cpp:14-62) */
FA_API fa_kernel_id_t fa_dispatch_select(int batch_heads, int seq_len, int head_dim, int causal, int window);

/* replaces fa_kernel_name, fa_sm120.h:150 */
FA_API const char* fa_kernel_name(fa_kernel_id_t id);

/* ---- additive extensions (no counterpart in the reference ABI) ---- */

/* All arguments of one forward call behind a single pointer (purego passes at
 * most a dozen scalars; goml wraps longer calls the same way,
 * backend/cuda/cublas_fp8.go:23-34).  v_descale multiplies O inside the kernel
 * so the fp16 output is already in real units (0 is treated as 1).
 * scale_q/scale_k/scale_v_dev: optional DEVICE pointers to one float each (the
 * scales a quantiser wrote); when non-NULL they multiply `scale` / `v_descale`
 * on the device, so no host round trip is needed between quantiser and attention. */
typedef struct {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    void* l_out; /* may be NULL */
    int batch_heads, seq_len, head_dim;
    int causal, window;
    float scale;
    float v_descale;
    const float* scale_q_dev;
    const float* scale_k_dev;
    const float* scale_v_dev;
    fa_stream_t stream;
} fa_forward_args_t;

FA_API fa_status_t fa_forward_ex(fa_ctx_t* ctx, const fa_forward_args_t* args);

/* No counterpart in the reference: an attention forward that allocates nothing.
 * The other entry points draw their scratch (an fp16 copy of V, 2*BH*S*D bytes) from a
 * memory pool.  This one is for callers that may not touch the allocator at all — code
 * embedded in a framework that reserved the whole GPU up front and forbids later
 * cudaMalloc-family calls, or real-time / safety-certified processes whose device memory
 * map is frozen after start-up.  Its scratch is a fixed 32 MiB device array inside the
 * library (held by every GPU that loads it, until exit), so one call is limited to
 *     batch_heads * seq_len * head_dim <= 16 Mi (16 777 216) elements;
 * larger problems return FA_ERR_UNSUPPORTED_SHAPE with a message (split the batch, or use
 * fa_forward_ex).  Arguments and results are those of fa_forward_ex (same kernels); no
 * context is needed.  err/err_len: optional caller buffer that receives a message on failure.
 * The array is shared by all calls on a GPU: calls whose GPU work overlaps race on it — use
 * one stream or serialise.  The first call on each device performs a one-time set-up
 * (device address of the array, kernel attributes); make it before any stream capture.
 * Where the CUDA runtime loads modules lazily, that first call is also the moment the driver
 * reserves the 32 MiB on that GPU: a process that freezes its memory map must make the first
 * call (a one-row problem will do) during start-up, not merely before capture. */
FA_API fa_status_t fa_forward_noalloc(const fa_forward_args_t* args, char* err, int err_len);

/* No counterpart in the reference: fa_device_status for callers without a context (users of
 * fa_forward_noalloc; fa_create would create a memory pool).  Synchronises the current device
 * and returns, and clears, the first bounded-wait expiry code an attention kernel recorded:
 * 0 = none, > 0 = the code, < 0 = a CUDA error code negated.  Allocates nothing. */
FA_API int fa_noalloc_device_status(void);

/* No counterpart in the reference (designed on paper there, runs/reports/F1_HF_INFERENCE_recon.md:55-68,163): the
 * decode step of quantised inference — one new token per sequence attends to an FP8 KV cache, with grouped-query
 * heads.  q [batch, q_heads, head_dim] e4m3; k_cache, v_cache [batch, kv_heads, s_max, head_dim] e4m3 (the layout
 * fa_forward reads with batch_heads = batch * kv_heads and seq_len = s_max, so a cache filled during prefill is used
 * as is); o [batch, q_heads, head_dim] fp16; l_out [batch, q_heads] fp32 natural-log LSE or NULL.  Query head h uses
 * kv head h / (q_heads / kv_heads); q_heads / kv_heads must be an integer <= 16.  Sequence b sees keys
 * [0, seq_lens[b]) (seq_lens: batch int32 values on the device, clamped to [0, s_max]) or, when seq_lens is NULL,
 * keys [0, seq_len).  scale = softmax_scale * scale_Q * scale_K, v_descale and the optional device scale pointers as
 * in fa_forward_ex.  A sequence with no visible key gets O = 0 and LSE = -inf.  HBM-bound: every cached key and value
 * is read once.  Cache bytes at or past a sequence's length are never used, whatever they hold.
 * Paged cache (block_table != NULL): k_cache, v_cache are pools [num_pages, kv_heads, page_size, head_dim], page_size
 * a multiple of 64; block_table [batch, max_pages_per_seq] int32 on the device gives the pool page that holds keys
 * [j * page_size, (j+1) * page_size) of sequence b at block_table[b * max_pages_per_seq + j]; s_max is then
 * max_pages_per_seq * page_size (the field is ignored).  Only entries below ceil(seq_len / page_size) are read; an
 * entry outside [0, num_pages) reads nothing and its keys count as zeros.  Zero the struct before filling it: with
 * block_table == NULL the last four fields are ignored. */
typedef struct fa_decode_args {
    const void* q;
    const void* k_cache;
    const void* v_cache;
    void* o;
    void* l_out;
    const int* seq_lens;
    int batch, q_heads, kv_heads, head_dim;
    int s_max, seq_len;
    float scale;
    float v_descale;
    const float* scale_q_dev;
    const float* scale_k_dev;
    const float* scale_v_dev;
    fa_stream_t stream;
    const int* block_table;
    int page_size;
    int max_pages_per_seq;
    int num_pages;
} fa_decode_args_t;

FA_API fa_status_t fa_decode(fa_ctx_t* ctx, const fa_decode_args_t* args);

/* Synchronises the context's device and reports whether any attention kernel
 * recorded a bounded-wait expiry since the last call: FA_OK, or FA_ERR_INTERNAL
 * with the code in fa_last_cuda_error. */
FA_API fa_status_t fa_device_status(fa_ctx_t* ctx);

/* No counterpart in the reference: self-test of the bounded waits.  Launches one warp that waits, with a 1 ms budget,
 * on a barrier nothing ever arrives at; the wait gives up and the kernel returns after latching code 0x2F0 the way an
 * attention kernel's teardown would.  The next fa_device_status() must therefore return FA_ERR_INTERNAL with
 * "device status 0x2f0" as the message, and the one after that FA_OK.  No operand memory, TMA or tensor memory is
 * touched; the GPU context stays usable. */
FA_API fa_status_t fa_selftest_wait_expiry(fa_ctx_t* ctx, fa_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* FA_SM120_H_ */
