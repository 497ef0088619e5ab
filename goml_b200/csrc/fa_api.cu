// fa_api.cu — context lifecycle, argument validation and the C entry points of
// libfa_sm120.so (the ABI of goml's libs/fa_sm120/src/fa_ctx.cu:55-235).
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "../../include/fa_sm120.h"
#include "fa_fwd_sm100.h"

struct fa_ctx {
    int device;
    int cc_major, cc_minor;
    bool arch_ok;
    // Stream-ordered pool the per-call scratch (the fp16 copy of V) is drawn from and
    // returned to; freed blocks stay cached in the pool, so steady-state calls do not
    // reach the driver allocator.  Owned by the context, destroyed with it.
    cudaMemPool_t pool;
    bool has_pool;
    char last_err[256];
};

namespace {

void set_err(fa_ctx_t* c, const char* fmt, const char* a = "", const char* b = "") {
    if (c) snprintf(c->last_err, sizeof(c->last_err), fmt, a, b);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Checks shared by every forward entry.  `who` prefixes messages.
fa_status_t validate(fa_ctx_t* c, const char* who, const void* q, const void* k, const void* v, const void* o,
                     int bh, int sl, int hd, int causal, int window, const void* l_out = nullptr) {
    if (!c->arch_ok || !c->has_pool) { set_err(c, "%s: context was created on an unsupported GPU", who); return FA_ERR_UNSUPPORTED_ARCH; }
    if (!q || !k || !v || !o) { set_err(c, "%s: null pointer in q/k/v/o", who); return FA_ERR_INVALID_ARG; }
    if (bh <= 0 || sl <= 0) { set_err(c, "%s: bh/sl must be > 0", who); return FA_ERR_INVALID_ARG; }
    if (hd != 64 && hd != 128) { set_err(c, "%s: head_dim must be 64 or 128", who); return FA_ERR_UNSUPPORTED_HD; }
    if (window < 0 || window > sl) { set_err(c, "%s: window must be in [0, seq_len]", who); return FA_ERR_INVALID_ARG; }
    if (causal != 0 && causal != 1) { set_err(c, "%s: causal must be 0 or 1", who); return FA_ERR_INVALID_ARG; }
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) {
        set_err(c, "%s: q/k/v/o must be 16-byte aligned", who);
        return FA_ERR_INVALID_ARG;
    }
    if (reinterpret_cast<uintptr_t>(l_out) & 3) { set_err(c, "%s: l_out must be 4-byte aligned", who); return FA_ERR_INVALID_ARG; }
    if (fa_dispatch_select(bh, sl, hd, causal, window) == FA_KERNEL_NONE) {
        set_err(c, "%s: no kernel matches this configuration", who);
        return FA_ERR_UNSUPPORTED_SHAPE;
    }
    return FA_OK;
}

fa_status_t run(fa_ctx_t* c, const char* who, const fa_sm100::LaunchArgs& a) {
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) { set_err(c, "%s: cudaGetDevice: %s", who, cudaGetErrorString(e)); return FA_ERR_CUDA; }
    if (cur != c->device) {
        // one context serves the device it was created on; the caller keeps that device current
        set_err(c, "%s: the calling thread's current device differs from the context's device", who);
        return FA_ERR_INVALID_ARG;
    }
    fa_sm100::LaunchArgs b = a;
    void* ws = nullptr;
    e = cudaMallocFromPoolAsync(&ws, fa_sm100::workspace_bytes(a.bh, a.sl, a.hd), c->pool, a.stream);
    if (e != cudaSuccess) {
        set_err(c, "%s: workspace allocation: %s", who, cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? FA_ERR_OOM : FA_ERR_CUDA;
    }
    b.v16_workspace = ws;
    e = fa_sm100::launch(b);
    const cudaError_t fe = cudaFreeAsync(ws, a.stream);  // stream-ordered: released after the kernel
    if (e != cudaSuccess) { set_err(c, "%s: launch: %s", who, cudaGetErrorString(e)); return FA_ERR_CUDA; }
    if (fe != cudaSuccess) { set_err(c, "%s: workspace release: %s", who, cudaGetErrorString(fe)); return FA_ERR_CUDA; }
    return FA_OK;
}

}  // namespace

extern "C" {

fa_status_t fa_create(fa_ctx_t** ctx_out) {
    if (!ctx_out) return FA_ERR_INVALID_ARG;
    *ctx_out = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return FA_ERR_CUDA;
    fa_ctx_t* c = new (std::nothrow) fa_ctx_t();
    if (!c) return FA_ERR_OOM;
    c->device = dev;
    c->last_err[0] = '\0';
    if (cudaDeviceGetAttribute(&c->cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&c->cc_minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
        delete c;
        return FA_ERR_CUDA;
    }
    c->arch_ok = (c->cc_major == 10);
    c->has_pool = false;
    if (c->arch_ok) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaError_t pe = cudaMemPoolCreate(&c->pool, &props);
        if (pe != cudaSuccess) {
            snprintf(c->last_err, sizeof(c->last_err), "fa_create: cudaMemPoolCreate: %s", cudaGetErrorString(pe));
            *ctx_out = c;
            return FA_ERR_CUDA;
        }
        unsigned long long keep = ~0ull;  // keep freed scratch cached in the pool
        cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &keep);
        c->has_pool = true;
    }
    *ctx_out = c;  // returned even on an unsupported GPU so the caller can read the reason
    if (!c->arch_ok) {
        snprintf(c->last_err, sizeof(c->last_err),
                 "GPU compute capability %d.%d is not sm_100a (need 10.x).", c->cc_major, c->cc_minor);
        return FA_ERR_UNSUPPORTED_ARCH;
    }
    return FA_OK;
}

fa_status_t fa_destroy(fa_ctx_t* ctx) {
    if (ctx && ctx->has_pool) cudaMemPoolDestroy(ctx->pool);  // pending frees complete first (stream-ordered)
    delete ctx;
    return FA_OK;
}

const char* fa_version(void) { return "1.0.0+tcgen05-sm100a"; }

const char* fa_status_str(fa_status_t s) {
    switch (s) {
        case FA_OK: return "OK";
        case FA_ERR_INVALID_ARG: return "invalid argument";
        case FA_ERR_UNSUPPORTED_ARCH: return "unsupported GPU arch (need sm_100a)";
        case FA_ERR_UNSUPPORTED_HD: return "unsupported head_dim (need 64 or 128)";
        case FA_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
        case FA_ERR_CUDA: return "CUDA runtime error";
        case FA_ERR_OOM: return "out of memory";
        case FA_ERR_INTERNAL: return "internal error";
    }
    return "unknown";
}

const char* fa_last_cuda_error(fa_ctx_t* ctx) { return ctx ? ctx->last_err : ""; }

fa_status_t fa_forward_train(fa_ctx_t* ctx, const void* q, const void* k, const void* v, void* o, void* l_out,
                             int bh, int sl, int hd, int causal, int window, float scale, fa_stream_t stream) {
    if (!ctx) return FA_ERR_INVALID_ARG;
    fa_status_t s = validate(ctx, "fa_forward_train", q, k, v, o, bh, sl, hd, causal, window, l_out);
    if (s != FA_OK) return s;
    fa_sm100::LaunchArgs a{};
    a.q = q; a.k = k; a.v = v; a.o = o; a.lse = static_cast<float*>(l_out);
    a.bh = bh; a.sl = sl; a.hd = hd; a.causal = causal; a.window = window;
    a.scale = scale; a.v_descale = 1.0f;
    a.stream = reinterpret_cast<cudaStream_t>(stream);
    return run(ctx, "fa_forward_train", a);
}

fa_status_t fa_forward(fa_ctx_t* ctx, const void* q, const void* k, const void* v, void* o, int bh, int sl, int hd,
                       int causal, int window, float scale, fa_stream_t stream) {
    if (!ctx) return FA_ERR_INVALID_ARG;
    fa_status_t s = validate(ctx, "fa_forward", q, k, v, o, bh, sl, hd, causal, window);
    if (s != FA_OK) return s;
    fa_sm100::LaunchArgs a{};
    a.q = q; a.k = k; a.v = v; a.o = o; a.lse = nullptr;
    a.bh = bh; a.sl = sl; a.hd = hd; a.causal = causal; a.window = window;
    a.scale = scale; a.v_descale = 1.0f;
    a.stream = reinterpret_cast<cudaStream_t>(stream);
    return run(ctx, "fa_forward", a);
}

fa_status_t fa_forward_ex(fa_ctx_t* ctx, const fa_forward_args_t* g) {
    if (!ctx) return FA_ERR_INVALID_ARG;
    if (!g) { set_err(ctx, "%s: null argument block", "fa_forward_ex"); return FA_ERR_INVALID_ARG; }
    fa_status_t s = validate(ctx, "fa_forward_ex", g->q, g->k, g->v, g->o, g->batch_heads, g->seq_len, g->head_dim,
                             g->causal, g->window, g->l_out);
    if (s != FA_OK) return s;
    fa_sm100::LaunchArgs a{};
    a.q = g->q; a.k = g->k; a.v = g->v; a.o = g->o; a.lse = static_cast<float*>(g->l_out);
    a.bh = g->batch_heads; a.sl = g->seq_len; a.hd = g->head_dim; a.causal = g->causal; a.window = g->window;
    a.scale = g->scale; a.v_descale = (g->v_descale == 0.0f) ? 1.0f : g->v_descale;
    a.scale_q_dev = g->scale_q_dev; a.scale_k_dev = g->scale_k_dev; a.scale_v_dev = g->scale_v_dev;
    a.stream = reinterpret_cast<cudaStream_t>(g->stream);
    return run(ctx, "fa_forward_ex", a);
}

fa_status_t fa_decode(fa_ctx_t* ctx, const fa_decode_args_t* g) {
    const char* who = "fa_decode";
    if (!ctx) return FA_ERR_INVALID_ARG;
    if (!g) { set_err(ctx, "%s: null argument block", who); return FA_ERR_INVALID_ARG; }
    if (!ctx->arch_ok || !ctx->has_pool) { set_err(ctx, "%s: context was created on an unsupported GPU", who); return FA_ERR_UNSUPPORTED_ARCH; }
    if (!g->q || !g->k_cache || !g->v_cache || !g->o) { set_err(ctx, "%s: null pointer in q/k_cache/v_cache/o", who); return FA_ERR_INVALID_ARG; }
    const bool paged = g->block_table != nullptr;
    if (paged && (g->page_size <= 0 || g->page_size % 64 != 0 || g->max_pages_per_seq <= 0 || g->num_pages <= 0 ||
                  (long long)g->page_size * g->max_pages_per_seq > 0x7fffffffLL)) {
        set_err(ctx, "%s: paged cache needs page_size a positive multiple of 64, max_pages_per_seq > 0 and num_pages > 0", who);
        return FA_ERR_INVALID_ARG;
    }
    const int s_max = paged ? g->page_size * g->max_pages_per_seq : g->s_max;
    if (g->batch <= 0 || g->q_heads <= 0 || g->kv_heads <= 0 || s_max <= 0) { set_err(ctx, "%s: batch/heads/s_max must be > 0", who); return FA_ERR_INVALID_ARG; }
    if (g->head_dim != 64 && g->head_dim != 128) { set_err(ctx, "%s: head_dim must be 64 or 128", who); return FA_ERR_UNSUPPORTED_HD; }
    if (g->q_heads % g->kv_heads != 0 || g->q_heads / g->kv_heads > 16) {
        set_err(ctx, "%s: q_heads must be a multiple of kv_heads with at most 16 query heads per kv head", who);
        return FA_ERR_UNSUPPORTED_SHAPE;
    }
    if (!g->seq_lens && (g->seq_len < 0 || g->seq_len > s_max)) { set_err(ctx, "%s: seq_len must be in [0, s_max]", who); return FA_ERR_INVALID_ARG; }
    if ((reinterpret_cast<uintptr_t>(g->q) & 3) || !aligned16(g->k_cache) || !aligned16(g->v_cache) || (reinterpret_cast<uintptr_t>(g->o) & 1)) {
        set_err(ctx, "%s: k_cache/v_cache must be 16-byte aligned, q 4-byte aligned", who);
        return FA_ERR_INVALID_ARG;
    }
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) { set_err(ctx, "%s: cudaGetDevice: %s", who, cudaGetErrorString(e)); return FA_ERR_CUDA; }
    if (cur != ctx->device) { set_err(ctx, "%s: the calling thread's current device differs from the context's device", who); return FA_ERR_INVALID_ARG; }
    fa_sm100::DecodeArgs a{};
    a.q = g->q; a.k_cache = g->k_cache; a.v_cache = g->v_cache; a.o = g->o; a.lse = static_cast<float*>(g->l_out);
    a.seq_lens = g->seq_lens;
    a.batch = g->batch; a.q_heads = g->q_heads; a.kv_heads = g->kv_heads; a.hd = g->head_dim;
    a.s_max = s_max; a.seq_len = g->seq_len;
    a.block_table = g->block_table; a.page_size = g->page_size; a.max_pages = g->max_pages_per_seq; a.num_pages = g->num_pages;
    a.scale = g->scale; a.v_descale = (g->v_descale == 0.0f) ? 1.0f : g->v_descale;
    a.scale_q_dev = g->scale_q_dev; a.scale_k_dev = g->scale_k_dev; a.scale_v_dev = g->scale_v_dev;
    a.stream = reinterpret_cast<cudaStream_t>(g->stream);
    const size_t ws_bytes = fa_sm100::decode_workspace_bytes(a.batch, a.kv_heads, a.hd, fa_sm100::decode_span(a));
    void* ws = nullptr;
    if (ws_bytes) {
        e = cudaMallocFromPoolAsync(&ws, ws_bytes, ctx->pool, a.stream);
        if (e != cudaSuccess) { set_err(ctx, "%s: workspace allocation: %s", who, cudaGetErrorString(e)); return e == cudaErrorMemoryAllocation ? FA_ERR_OOM : FA_ERR_CUDA; }
    }
    a.workspace = ws;
    e = fa_sm100::launch_decode(a);
    const cudaError_t fe = ws ? cudaFreeAsync(ws, a.stream) : cudaSuccess;  // stream-ordered: released after the kernels
    if (e != cudaSuccess) { set_err(ctx, "%s: launch: %s", who, cudaGetErrorString(e)); return FA_ERR_CUDA; }
    if (fe != cudaSuccess) { set_err(ctx, "%s: workspace release: %s", who, cudaGetErrorString(fe)); return FA_ERR_CUDA; }
    return FA_OK;
}

fa_status_t fa_selftest_wait_expiry(fa_ctx_t* ctx, fa_stream_t stream) {
    if (!ctx) return FA_ERR_INVALID_ARG;
    if (!ctx->arch_ok) { set_err(ctx, "%s: context was created on an unsupported GPU", "fa_selftest_wait_expiry"); return FA_ERR_UNSUPPORTED_ARCH; }
    const cudaError_t e = fa_sm100::launch_wait_expiry_selftest(reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_err(ctx, "%s: launch: %s", "fa_selftest_wait_expiry", cudaGetErrorString(e)); return FA_ERR_CUDA; }
    return FA_OK;
}

fa_status_t fa_device_status(fa_ctx_t* ctx) {
    if (!ctx) return FA_ERR_INVALID_ARG;
    const int code = fa_sm100::device_status();
    if (code == 0) return FA_OK;
    if (code < 0) {
        set_err(ctx, "%s: %s", "fa_device_status", cudaGetErrorString(static_cast<cudaError_t>(-code)));
        return FA_ERR_CUDA;
    }
    snprintf(ctx->last_err, sizeof(ctx->last_err), "a kernel wait ran out (device status 0x%x)", code);
    return FA_ERR_INTERNAL;
}

}  // extern "C"
