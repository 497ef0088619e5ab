// fa_fwd_sm100.h — internal launch interface between the C-ABI layer (fa_api.cu)
// and the sm_100a attention kernels (fa_fwd_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa_sm100 {

struct LaunchArgs {
    const void* q;      // [bh, sl, hd] e4m3
    const void* k;
    const void* v;
    void* o;            // [bh, sl, hd] fp16
    float* lse;         // [bh, sl] fp32 natural-log LSE, or nullptr
    void* v16_workspace = nullptr;  // workspace_bytes(bh, sl, hd) bytes, 128-byte aligned: fp16 copy of V
    int bh, sl, hd;     // hd in {64, 128}
    int causal, window;
    float scale;        // softmax_scale * scale_q * scale_k
    float v_descale;    // multiplies O (1 = output in decoded-V units, as the reference)
    const float* scale_q_dev = nullptr;  // optional device scalars multiplied into scale / v_descale
    const float* scale_k_dev = nullptr;
    const float* scale_v_dev = nullptr;
    cudaStream_t stream;
};

// Scratch the forward needs (an fp16 copy of V made by a pre-pass on the same stream).
size_t workspace_bytes(int bh, int sl, int hd);

// Launches on the calling thread's current device; asynchronous on a.stream.
cudaError_t launch(const LaunchArgs& a);

// ---- decode step: one new token per sequence against an FP8 KV cache, grouped-query heads (fa_decode_sm100.cu)
struct DecodeArgs {
    const void* q;         // [batch, q_heads, hd] e4m3
    const void* k_cache;   // [batch, kv_heads, s_max, hd] e4m3
    const void* v_cache;
    void* o;               // [batch, q_heads, hd] fp16
    float* lse;            // [batch, q_heads] or nullptr
    const int* seq_lens;   // [batch] on the device, or nullptr: every sequence has seq_len keys
    int batch, q_heads, kv_heads, hd, s_max, seq_len;
    float scale, v_descale;
    const float* scale_q_dev = nullptr;
    const float* scale_k_dev = nullptr;
    const float* scale_v_dev = nullptr;
    void* workspace = nullptr;  // decode_workspace_bytes(...) bytes (0 when one split suffices)
    cudaStream_t stream;
    // paged cache (block_table != nullptr): k_cache, v_cache are [num_pages, kv_heads, page_size, hd], page_size a
    // multiple of 64; block_table [batch, max_pages] holds the page of each page_size-key range of a sequence and
    // s_max = max_pages * page_size
    const int* block_table = nullptr;
    int page_size = 0, max_pages = 0, num_pages = 0;
};
// Longest key range any sequence can have in this call (s_max with per-sequence lengths, else seq_len).
inline int decode_span(const DecodeArgs& a) { return a.seq_lens ? a.s_max : a.seq_len; }
size_t decode_workspace_bytes(int batch, int kv_heads, int head_dim, int span);
cudaError_t launch_decode(const DecodeArgs& a);

// One warp that lets a 1 ms bounded wait run out on a barrier nothing arrives at and latches code 0x2F0.
cudaError_t launch_wait_expiry_selftest(cudaStream_t stream);

// Synchronises the device and returns (and clears) the first non-zero status
// code a kernel recorded (a wait that ran out), 0 if none, -cudaError on failure.
int device_status();

}  // namespace fa_sm100
