// goml_cuda.hpp — C++ host side above the C ABI, mirroring goml's Go package backend/cuda for this path.
//
// goml binds its CUDA libraries without cgo: `purego.Dlopen` + `RegisterLibFunc`
// (backend/cuda/fp8_gemm.go:27-41, backend/cuda/fa_forward.go:74-115) behind a library search
// (backend/cuda/arch.go:57-101).  This header does the same with dlopen/dlsym and keeps the names,
// argument meaning and error text of that package:
//
//   LibsDir / resolveLib                      arch.go:63-101
//   FP8GEMM(M,N,K,A,B,C,mode,stream)          fp8_gemm.go:52-62     ("fp8_gemm: CUDA error %d")
//   FALoad / FACreate / FAContext::ForwardTrain / Destroy / FAVersion / FAStatus strings
//                                             fa_forward.go:25-215  ("fa_forward_train: <status> (<message>)")
//   QuantizeF32ToF8E4M3 / ...Unit             the calls of internal/abjexam/battle_a_llm.go:476-494
// plus what goml lacks: the additive entry points (FP8GEMMScaled, ForwardEx) and a multi-GPU manager
// (one context + one stream per device; contiguous head / row-tile partitions).
//
// Pointers are raw device addresses (uintptr_t), as in the Go bindings.  Errors are thrown as
// goml::cuda::Error.  Header-only; link with -ldl and the CUDA runtime (for the device manager).
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/fa_sm120.h"
#include "../../include/fp8_block.h"   // fp8_decode_append_args_t (the functions are bound at run time, not linked)

namespace goml {
namespace cuda {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

namespace detail {
inline bool is_dir(const std::string& p) { struct stat st; return !p.empty() && stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }
inline bool is_file(const std::string& p) { struct stat st; return !p.empty() && stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode); }
inline std::string env(const char* k) { const char* v = getenv(k); return v ? v : ""; }
inline std::string exe_dir() {
    char buf[4096];
    ssize_t n = readlink("/proc/self/exe", buf, sizeof(buf) - 1);
    if (n <= 0) return "";
    buf[n] = 0;
    std::string s(buf);
    return s.substr(0, s.find_last_of('/'));
}
template <class Fn>
Fn sym(void* lib, const char* name) {
    void* p = dlsym(lib, name);
    if (!p) throw Error(std::string("dlsym ") + name + ": " + dlerror());
    return reinterpret_cast<Fn>(p);
}
}  // namespace detail

// Directory searched for the prebuilt libraries.  Priority (arch.go:57-82): $GOML_LIBS_DIR, ./libs,
// <executable dir>/libs, /usr/local/lib/goml; the first existing directory wins; "" if none.
inline std::string LibsDir() {
    char cwd[4096];
    std::vector<std::string> c = {detail::env("GOML_LIBS_DIR")};
    if (getcwd(cwd, sizeof(cwd))) c.push_back(std::string(cwd) + "/libs");
    if (!detail::exe_dir().empty()) c.push_back(detail::exe_dir() + "/libs");
    c.push_back("/usr/local/lib/goml");
    for (const auto& d : c)
        if (detail::is_dir(d)) return d;
    return "";
}
// Full path when the file exists in LibsDir(), else the bare name for the OS loader (arch.go:84-101).
inline std::string resolveLib(const std::string& name) {
    const std::string d = LibsDir();
    if (!d.empty() && detail::is_file(d + "/" + name)) return d + "/" + name;
    return name;
}

// ------------------------------------------------------------------------------------ FP8 GEMM
enum { ModeOriginal = 0, ModeSinglesync = 1 };
enum { FP8OutFP16 = 0, FP8OutBF16 = 1 };

namespace detail {
struct GemmLib {
    void* lib = nullptr;
    int (*gemm)(int, int, int, const void*, const void*, void*, int, void*) = nullptr;
    int (*original)(int, int, int, const void*, const void*, void*, void*) = nullptr;
    int (*ss)(int, int, int, const void*, const void*, void*, void*) = nullptr;
    int (*scaled)(int, int, int, const void*, const void*, void*, float, const float*, const float*, int, void*) = nullptr;
    int (*accumulate)(int, int, int, const void*, const void*, float*, float, const float*, const float*, void*) = nullptr;
    int (*swiglu)(int, int, int, const void*, const void*, void*, float, const float*, const float*, float*, void*) = nullptr;
    int (*fp8out)(int, int, int, const void*, const void*, void*, float, const float*, const float*, const float*, float*, void*) = nullptr;
    int (*status)() = nullptr;
    int (*mx)(int, int, int, const void*, const void*, const void*, const void*, void*, float, int, void*) = nullptr;
    size_t (*mx_scale_bytes)(int, int) = nullptr;
    int (*set_pairs)(int) = nullptr;
};
inline GemmLib& gemm_lib() {  // sync.Once-style (fp8_gemm.go:27-41)
    static GemmLib g;
    static std::once_flag once;
    static std::string err;
    std::call_once(once, [] {
        g.lib = dlopen(resolveLib("libfp8gemm.so").c_str(), RTLD_LAZY | RTLD_GLOBAL);
        if (!g.lib) { err = std::string("fp8gemm: dlopen: ") + dlerror(); return; }
        g.gemm = sym<decltype(g.gemm)>(g.lib, "fp8_gemm");
        g.original = sym<decltype(g.original)>(g.lib, "fp8_gemm_original");
        g.ss = sym<decltype(g.ss)>(g.lib, "fp8_gemm_singlesync");
        g.scaled = sym<decltype(g.scaled)>(g.lib, "fp8_gemm_scaled");
        g.accumulate = sym<decltype(g.accumulate)>(g.lib, "fp8_gemm_accumulate_f32");
        g.swiglu = sym<decltype(g.swiglu)>(g.lib, "fp8_gemm_swiglu");
        g.fp8out = sym<decltype(g.fp8out)>(g.lib, "fp8_gemm_fp8out");
        g.status = sym<decltype(g.status)>(g.lib, "fp8_gemm_device_status");
        g.mx = sym<decltype(g.mx)>(g.lib, "fp8_gemm_mx");
        g.mx_scale_bytes = sym<decltype(g.mx_scale_bytes)>(g.lib, "fp8_mx_scale_bytes");
        g.set_pairs = sym<decltype(g.set_pairs)>(g.lib, "fp8_gemm_set_tile_pairs");
    });
    if (!g.lib) throw Error(err);
    return g;
}
inline void* vp(uintptr_t p) { return reinterpret_cast<void*>(p); }
}  // namespace detail

// C[M,N] (fp16) = A[M,K] x B[N,K]^T on e4m3 device buffers (fp8_gemm.go:52-62).
inline void FP8GEMM(int M, int N, int K, uintptr_t A, uintptr_t B, uintptr_t C, int mode, uintptr_t stream) {
    const int rc = detail::gemm_lib().gemm(M, N, K, detail::vp(A), detail::vp(B), detail::vp(C), mode, detail::vp(stream));
    if (rc != 0) throw Error("fp8_gemm: CUDA error " + std::to_string(rc));
}
// C = alpha * (*scaleA) * (*scaleB) * A x B^T; scale pointers are device addresses or 0.
inline void FP8GEMMScaled(int M, int N, int K, uintptr_t A, uintptr_t B, uintptr_t C, float alpha, uintptr_t scaleA,
                          uintptr_t scaleB, int outDType, uintptr_t stream) {
    const int rc = detail::gemm_lib().scaled(M, N, K, detail::vp(A), detail::vp(B), detail::vp(C), alpha,
                                             reinterpret_cast<const float*>(scaleA), reinterpret_cast<const float*>(scaleB),
                                             outDType, detail::vp(stream));
    if (rc != 0) throw Error("fp8_gemm_scaled: CUDA error " + std::to_string(rc));
}
// X (fp32 [M,N]) += alpha * (*scaleA) * (*scaleB) * A x B^T: the residual update of a decoder block in the epilogue.
inline void FP8GEMMAccumulateF32(int M, int N, int K, uintptr_t A, uintptr_t B, uintptr_t X, float alpha, uintptr_t scaleA,
                                 uintptr_t scaleB, uintptr_t stream) {
    const int rc = detail::gemm_lib().accumulate(M, N, K, detail::vp(A), detail::vp(B), reinterpret_cast<float*>(X), alpha,
                                                 reinterpret_cast<const float*>(scaleA), reinterpret_cast<const float*>(scaleB),
                                                 detail::vp(stream));
    if (rc != 0) throw Error("fp8_gemm_accumulate_f32: CUDA error " + std::to_string(rc));
}
// H (bf16 [M,F]) = silu(g) * u, [g | u] = alpha * (*scaleA) * (*scaleB) * A x Binterleaved^T; max|H| -> *amaxOut.
// Binterleaved: per 32 feed-forward columns the 32 gate rows then the 32 up rows (InterleaveGateUp below).
inline void FP8GEMMSwiGLU(int M, int F, int K, uintptr_t A, uintptr_t Binterleaved, uintptr_t H, float alpha, uintptr_t scaleA,
                          uintptr_t scaleB, uintptr_t amaxOut, uintptr_t stream) {
    const int rc = detail::gemm_lib().swiglu(M, F, K, detail::vp(A), detail::vp(Binterleaved), detail::vp(H), alpha,
                                             reinterpret_cast<const float*>(scaleA), reinterpret_cast<const float*>(scaleB),
                                             reinterpret_cast<float*>(amaxOut), detail::vp(stream));
    if (rc != 0) throw Error("fp8_gemm_swiglu: CUDA error " + std::to_string(rc));
}
// D (e4m3 [M,N]) = e4m3((*scaleD) * v), v = alpha * (*scaleA) * (*scaleB) * A x B^T; max|v| -> *amaxD (0: not wanted).
// The delayed-scaling epilogue of fp8_matmul_fp8out (libs1/cublas_lt_wrapper_v3.c:220-229).
inline void FP8GEMMFP8Out(int M, int N, int K, uintptr_t A, uintptr_t B, uintptr_t D, float alpha, uintptr_t scaleA,
                          uintptr_t scaleB, uintptr_t scaleD, uintptr_t amaxD, uintptr_t stream) {
    const int rc = detail::gemm_lib().fp8out(M, N, K, detail::vp(A), detail::vp(B), detail::vp(D), alpha,
                                             reinterpret_cast<const float*>(scaleA), reinterpret_cast<const float*>(scaleB),
                                             reinterpret_cast<const float*>(scaleD), reinterpret_cast<float*>(amaxD),
                                             detail::vp(stream));
    if (rc != 0) throw Error("fp8_gemm_fp8out: CUDA error " + std::to_string(rc));
}
// Host-side weight preparation for FP8GEMMSwiGLU: codes [2F, K] (gate rows first) -> [2*Fp, K], Fp = F rounded up to 32:
// per 32 feed-forward columns the 32 gate rows, then the 32 up rows; rows past F are zero.
inline std::vector<uint8_t> InterleaveGateUp(const std::vector<uint8_t>& gateUp, int F, int K) {
    const int Fp = (F + 31) / 32 * 32;
    std::vector<uint8_t> out((size_t)2 * Fp * K, 0);
    for (int col = 0; col < F; col++) {
        const size_t dst = (size_t)(64 * (col / 32) + col % 32) * K;
        std::copy(gateUp.begin() + (size_t)col * K, gateUp.begin() + (size_t)(col + 1) * K, out.begin() + dst);
        std::copy(gateUp.begin() + (size_t)(F + col) * K, gateUp.begin() + (size_t)(F + col + 1) * K, out.begin() + dst + (size_t)32 * K);
    }
    return out;
}
inline int FP8GEMMDeviceStatus() { return detail::gemm_lib().status(); }

// Block-scaled ("MXFP8") GEMM: e4m3 codes with one ue8m0 scale per 32 K elements of every row of A and of B (the arrays
// QuantizeMXF32 writes); C = alpha * sum over blocks of 2^(ea + eb) * A_kb . B_kb, fp16 / bf16 out.  K % 128 == 0.
inline void FP8GEMMMX(int M, int N, int K, uintptr_t A, uintptr_t scaleA, uintptr_t B, uintptr_t scaleB, uintptr_t C, float alpha,
                      int outDType, uintptr_t stream) {
    const int rc = detail::gemm_lib().mx(M, N, K, detail::vp(A), detail::vp(scaleA), detail::vp(B), detail::vp(scaleB), detail::vp(C), alpha,
                                         outDType, detail::vp(stream));
    if (rc != 0) throw Error("fp8_gemm_mx: CUDA error " + std::to_string(rc));
}
inline size_t MXScaleBytes(int rows, int K) { return detail::gemm_lib().mx_scale_bytes(rows, K); }
// -1 = tile pairs chosen per problem (default), 0 = single tiles only (bit-identical results)
inline void FP8GEMMSetTilePairs(int mode) {
    const int rc = detail::gemm_lib().set_pairs(mode);
    if (rc != 0) throw Error("fp8_gemm_set_tile_pairs: CUDA error " + std::to_string(rc));
}

// ----------------------------------------------------------------------------------- attention
using FAStatus = fa_status_t;

namespace detail {
struct FaLib {
    void* lib = nullptr;
    decltype(&fa_create) create = nullptr;
    decltype(&fa_destroy) destroy = nullptr;
    decltype(&fa_version) version = nullptr;
    decltype(&fa_status_str) status_str = nullptr;
    decltype(&fa_last_cuda_error) last_err = nullptr;
    decltype(&fa_forward) forward = nullptr;
    decltype(&fa_forward_train) forward_train = nullptr;
    decltype(&fa_forward_ex) forward_ex = nullptr;
    decltype(&fa_decode) decode = nullptr;
    decltype(&fa_dispatch_select) dispatch = nullptr;
    decltype(&fa_kernel_name) kernel_name = nullptr;
    decltype(&fa_device_status) device_status = nullptr;
    decltype(&fa_forward_noalloc) forward_noalloc = nullptr;
    decltype(&fa_noalloc_device_status) noalloc_status = nullptr;
};
inline FaLib& fa_lib() {
    static FaLib f;
    static std::once_flag once;
    static std::string err;
    std::call_once(once, [] {
        // search order of fa_forward.go:76-98
        std::vector<std::string> c;
        if (!env("GOML_FA_LIB").empty()) c.push_back(env("GOML_FA_LIB"));
        c.push_back(resolveLib("libfa_sm120.so"));
        c.push_back("libs/fa_sm120/libfa_sm120.so");
        c.push_back("./libfa_sm120.so");
        c.push_back("/usr/local/lib/libfa_sm120.so");
        std::string last;
        for (const auto& p : c) {
            if (p.find('/') != std::string::npos && !is_file(p)) continue;
            f.lib = dlopen(p.c_str(), RTLD_LAZY);
            if (f.lib) break;
            last = dlerror();
        }
        if (!f.lib) { err = "fa: dlopen libfa_sm120.so failed (" + last + "); set GOML_FA_LIB"; return; }
        f.create = sym<decltype(f.create)>(f.lib, "fa_create");
        f.destroy = sym<decltype(f.destroy)>(f.lib, "fa_destroy");
        f.version = sym<decltype(f.version)>(f.lib, "fa_version");
        f.status_str = sym<decltype(f.status_str)>(f.lib, "fa_status_str");
        f.last_err = sym<decltype(f.last_err)>(f.lib, "fa_last_cuda_error");
        f.forward = sym<decltype(f.forward)>(f.lib, "fa_forward");
        f.forward_train = sym<decltype(f.forward_train)>(f.lib, "fa_forward_train");
        f.forward_ex = sym<decltype(f.forward_ex)>(f.lib, "fa_forward_ex");
        f.decode = sym<decltype(f.decode)>(f.lib, "fa_decode");
        f.dispatch = sym<decltype(f.dispatch)>(f.lib, "fa_dispatch_select");
        f.kernel_name = sym<decltype(f.kernel_name)>(f.lib, "fa_kernel_name");
        f.device_status = sym<decltype(f.device_status)>(f.lib, "fa_device_status");
        f.forward_noalloc = sym<decltype(f.forward_noalloc)>(f.lib, "fa_forward_noalloc");
        f.noalloc_status = sym<decltype(f.noalloc_status)>(f.lib, "fa_noalloc_device_status");
    });
    if (!f.lib) throw Error(err);
    return f;
}
}  // namespace detail

inline void FALoad() { detail::fa_lib(); }
inline std::string FAVersion() { return detail::fa_lib().version(); }
inline std::string FAStatusString(FAStatus s) { return detail::fa_lib().status_str(s); }
inline int FADispatchSelect(int bh, int sl, int hd, int causal, int window) { return detail::fa_lib().dispatch(bh, sl, hd, causal, window); }

// Opaque handle; one per GPU (the device current when it was created).
class FAContext {
public:
    // Create an FA context on the current device.  As fa_forward.go:123-142: when the library hands back a
    // context together with an error, its message is read and the context destroyed.
    static std::unique_ptr<FAContext> FACreate() {
        auto& L = detail::fa_lib();
        fa_ctx_t* p = nullptr;
        const FAStatus st = L.create(&p);
        if (st != FA_OK) {
            std::string msg = "fa_create: " + std::string(L.status_str(st));
            if (p) { msg += " (" + std::string(L.last_err(p)) + ")"; L.destroy(p); }
            throw Error(msg);
        }
        return std::unique_ptr<FAContext>(new FAContext(p));
    }
    ~FAContext() { Destroy(); }
    void Destroy() { if (ptr_) { detail::fa_lib().destroy(ptr_); ptr_ = nullptr; } }

    // fa_forward.go:161-183.  q,k,v: e4m3 [bh,sl,hd]; o: fp16; lOut: fp32 [bh,sl] or 0.
    void ForwardTrain(uintptr_t q, uintptr_t k, uintptr_t v, uintptr_t o, uintptr_t lOut, int bh, int sl, int hd, int causal,
                      int window, float scale, uintptr_t stream) {
        check("FAContext.ForwardTrain");
        const FAStatus st = detail::fa_lib().forward_train(ptr_, detail::vp(q), detail::vp(k), detail::vp(v), detail::vp(o),
                                                           detail::vp(lOut), bh, sl, hd, causal, window, scale,
                                                           reinterpret_cast<fa_stream_t>(stream));
        if (st != FA_OK) fail("fa_forward_train", st);
    }
    void Forward(uintptr_t q, uintptr_t k, uintptr_t v, uintptr_t o, int bh, int sl, int hd, int causal, int window, float scale,
                 uintptr_t stream) {
        check("FAContext.Forward");
        const FAStatus st = detail::fa_lib().forward(ptr_, detail::vp(q), detail::vp(k), detail::vp(v), detail::vp(o), bh, sl, hd,
                                                     causal, window, scale, reinterpret_cast<fa_stream_t>(stream));
        if (st != FA_OK) fail("fa_forward", st);
    }
    void ForwardEx(const fa_forward_args_t& a) {
        check("FAContext.ForwardEx");
        const FAStatus st = detail::fa_lib().forward_ex(ptr_, &a);
        if (st != FA_OK) fail("fa_forward_ex", st);
    }    // One new token per sequence against an e4m3 KV cache, grouped-query heads (no counterpart in goml yet).
    void Decode(const fa_decode_args_t& a) {
        check("FAContext.Decode");
        const FAStatus st = detail::fa_lib().decode(ptr_, &a);
        if (st != FA_OK) fail("fa_decode", st);
    }

    void DeviceStatus() {
        const FAStatus st = detail::fa_lib().device_status(ptr_);
        if (st != FA_OK) fail("fa_device_status", st);
    }

private:
    explicit FAContext(fa_ctx_t* p) : ptr_(p) {}
    void check(const char* who) const { if (!ptr_) throw Error(std::string(who) + ": nil ctx"); }
    void fail(const char* entry, FAStatus st) const {
        auto& L = detail::fa_lib();
        throw Error(std::string(entry) + ": " + L.status_str(st) + " (" + L.last_err(ptr_) + ")");
    }
    fa_ctx_t* ptr_;
};

// Attention forward for callers that may not allocate (a process whose device memory map is frozen after start-up, code
// inside a framework that reserved the whole GPU): no context, scratch in a fixed 32 MiB array inside the library, so
// batch_heads * seq_len * head_dim <= 16 Mi per call.  Calls that overlap on the GPU share that array: one stream.
inline void FAForwardNoAlloc(const fa_forward_args_t& a) {
    char msg[256] = {0};
    const FAStatus st = detail::fa_lib().forward_noalloc(&a, msg, (int)sizeof(msg));
    if (st != FA_OK) throw Error(std::string("fa_forward_noalloc: ") + detail::fa_lib().status_str(st) + " (" + msg + ")");
}
// fa_device_status for callers without a context: 0, a kernel's wait-expiry code, or a negated CUDA error.
inline int FANoAllocDeviceStatus() { return detail::fa_lib().noalloc_status(); }

// ----------------------------------------------------------------------------------- quantiser
namespace detail {
struct QuantLib {
    void* lib = nullptr;
    int (*quant)(const float*, uint8_t*, float*, float*, size_t, int, void*) = nullptr;
    int (*quant_fp16)(const void*, void*, float*, int) = nullptr;
    int (*quant_mx)(const float*, uint8_t*, uint8_t*, int, int, void*) = nullptr;
};
inline QuantLib& quant_lib() {
    static QuantLib q;
    static std::once_flag once;
    static std::string err;
    std::call_once(once, [] {
        q.lib = dlopen(resolveLib("libfp8quant.so").c_str(), RTLD_LAZY);
        if (!q.lib) { err = std::string("fp8quant: dlopen: ") + dlerror(); return; }
        q.quant = sym<decltype(q.quant)>(q.lib, "fp8_quantize_f32");
        q.quant_fp16 = sym<decltype(q.quant_fp16)>(q.lib, "fp8_quantize_fp16");
        q.quant_mx = sym<decltype(q.quant_mx)>(q.lib, "fp8_quantize_mx_f32");
    });
    if (!q.lib) throw Error(err);
    return q;
}
inline void quantize(uintptr_t src, uintptr_t dst, uintptr_t scale, uintptr_t amax, size_t n, int conv, uintptr_t stream) {
    const int rc = quant_lib().quant(reinterpret_cast<const float*>(src), reinterpret_cast<uint8_t*>(dst),
                                     reinterpret_cast<float*>(scale), reinterpret_cast<float*>(amax), n, conv, vp(stream));
    if (rc != 0) throw Error("fp8_quantize_f32: CUDA error " + std::to_string(rc));
}
}  // namespace detail
// scale = amax/448 (libs1/fp8_quantize_v2.cu:91)
inline void QuantizeF32ToF8E4M3(uintptr_t src, uintptr_t dst, uintptr_t scale, uintptr_t amax, size_t n, uintptr_t stream = 0) {
    detail::quantize(src, dst, scale, amax, n, 0, stream);
}
// scale = amax: decoded magnitudes <= 1 (battle_a_llm.go:476)
inline void QuantizeF32ToF8E4M3Unit(uintptr_t src, uintptr_t dst, uintptr_t scale, uintptr_t amax, size_t n, uintptr_t stream = 0) {
    detail::quantize(src, dst, scale, amax, n, 1, stream);
}

// fp8_quantize_fp16 of libs1/fp8_quantize_v2.cu:176-204: FP16 source, scale = amax/448, legacy default stream
inline void QuantizeFP16(uintptr_t src, uintptr_t dst, uintptr_t scale, int n) {
    const int rc = detail::quant_lib().quant_fp16(detail::vp(src), detail::vp(dst), reinterpret_cast<float*>(scale), n);
    if (rc != 0) throw Error("fp8_quantize_fp16: CUDA error " + std::to_string(rc));
}
// [rows, K] fp32 -> e4m3 codes + ue8m0 block scales (one per 32 elements), the operand format of FP8GEMMMX
inline void QuantizeMXF32(uintptr_t src, uintptr_t codes, uintptr_t scales, int rows, int K, uintptr_t stream = 0) {
    const int rc = detail::quant_lib().quant_mx(reinterpret_cast<const float*>(src), reinterpret_cast<uint8_t*>(codes),
                                                reinterpret_cast<uint8_t*>(scales), rows, K, detail::vp(stream));
    if (rc != 0) throw Error("fp8_quantize_mx_f32: CUDA error " + std::to_string(rc));
}

// ----------------------------------------------------------------------- decoder-block glue
// libfp8block.so: RMSNorm (+ residual), half-split RoPE + head permute of Q/K/V, head permute of the attention
// output, SwiGLU and the residual add, each fused with the quantiser of its consumer.  They take the place of
// libtransformer.so's rmsnorm_forward / rope_forward / swiglu_forward (libs/transformer_kernels.cu:384-438)
// followed by separate quantiser launches (internal/abjexam/battle_a_llm.go:380-494).
namespace detail {
struct BlockLib {
    void* lib = nullptr;
    int (*rope_table)(float*, float*, int, int, float, void*) = nullptr;
    int (*rmsnorm_q)(const float*, const void*, float*, const float*, uint8_t*, float*, float*, float*, int, int, float, void*) = nullptr;
    int (*rope_q)(const void*, const float*, const float*, uint8_t*, uint8_t*, uint8_t*, float*, float*, int, int, int, int, void*) = nullptr;
    int (*permute_q)(const void*, uint8_t*, float*, float*, int, int, int, int, void*) = nullptr;
    int (*swiglu_q)(const void*, uint8_t*, float*, float*, int, int, void*) = nullptr;
    int (*quant_bf16)(const void*, uint8_t*, float*, const float*, size_t, void*) = nullptr;
    int (*residual_add)(float*, const void*, size_t, void*) = nullptr;
    int (*decode_append)(const fp8_decode_append_args_t*) = nullptr;
};
inline BlockLib& block_lib() {
    static BlockLib b;
    static std::once_flag once;
    static std::string err;
    std::call_once(once, [] {
        b.lib = dlopen(resolveLib("libfp8block.so").c_str(), RTLD_LAZY);
        if (!b.lib) { err = std::string("fp8block: dlopen: ") + dlerror(); return; }
        b.rope_table = sym<decltype(b.rope_table)>(b.lib, "fp8_rope_table");
        b.rmsnorm_q = sym<decltype(b.rmsnorm_q)>(b.lib, "fp8_rmsnorm_quantize");
        b.rope_q = sym<decltype(b.rope_q)>(b.lib, "fp8_rope_quantize_qkv");
        b.permute_q = sym<decltype(b.permute_q)>(b.lib, "fp8_permute_quantize_heads");
        b.swiglu_q = sym<decltype(b.swiglu_q)>(b.lib, "fp8_swiglu_quantize");
        b.quant_bf16 = sym<decltype(b.quant_bf16)>(b.lib, "fp8_quantize_bf16");
        b.residual_add = sym<decltype(b.residual_add)>(b.lib, "fp8_residual_add");
        b.decode_append = sym<decltype(b.decode_append)>(b.lib, "fp8_decode_rope_append");
    });
    if (!b.lib) throw Error(err);
    return b;
}
inline void block_check(const char* what, int rc) {
    if (rc != 0) throw Error(std::string(what) + ": CUDA error " + std::to_string(rc));
}
template <class T>
inline T* tp(uintptr_t p) { return reinterpret_cast<T*>(p); }
}  // namespace detail
inline void RopeTable(uintptr_t cos, uintptr_t sin, int seqLen, int headDim, float theta, uintptr_t stream = 0) {
    detail::block_check("fp8_rope_table", detail::block_lib().rope_table(detail::tp<float>(cos), detail::tp<float>(sin), seqLen, headDim, theta, detail::vp(stream)));
}
// residualBF16 and hOut may be 0; hOut may equal x (the residual stream is then updated in place)
inline void RMSNormQuantize(uintptr_t x, uintptr_t residualBF16, uintptr_t hOut, uintptr_t gamma, uintptr_t q, uintptr_t scale, uintptr_t amax,
                            uintptr_t rstdWs, int rows, int hidden, float eps, uintptr_t stream = 0) {
    detail::block_check("fp8_rmsnorm_quantize",
                        detail::block_lib().rmsnorm_q(detail::tp<const float>(x), detail::vp(residualBF16), detail::tp<float>(hOut), detail::tp<const float>(gamma),
                                                      detail::tp<uint8_t>(q), detail::tp<float>(scale), detail::tp<float>(amax), detail::tp<float>(rstdWs), rows,
                                                      hidden, eps, detail::vp(stream)));
}
inline void RopeQuantizeQKV(uintptr_t qkvBF16, uintptr_t cos, uintptr_t sin, uintptr_t q, uintptr_t k, uintptr_t v, uintptr_t scales, uintptr_t amaxes,
                            int batch, int seqLen, int heads, int headDim, uintptr_t stream = 0) {
    detail::block_check("fp8_rope_quantize_qkv",
                        detail::block_lib().rope_q(detail::vp(qkvBF16), detail::tp<const float>(cos), detail::tp<const float>(sin), detail::tp<uint8_t>(q),
                                                   detail::tp<uint8_t>(k), detail::tp<uint8_t>(v), detail::tp<float>(scales), detail::tp<float>(amaxes), batch,
                                                   seqLen, heads, headDim, detail::vp(stream)));
}
inline void PermuteQuantizeHeads(uintptr_t oFP16, uintptr_t q, uintptr_t scale, uintptr_t amax, int batch, int seqLen, int heads, int headDim,
                                 uintptr_t stream = 0) {
    detail::block_check("fp8_permute_quantize_heads", detail::block_lib().permute_q(detail::vp(oFP16), detail::tp<uint8_t>(q), detail::tp<float>(scale),
                                                                                    detail::tp<float>(amax), batch, seqLen, heads, headDim, detail::vp(stream)));
}
inline void SwiGLUQuantize(uintptr_t gateUpBF16, uintptr_t q, uintptr_t scale, uintptr_t amax, int rows, int ffnHidden, uintptr_t stream = 0) {
    detail::block_check("fp8_swiglu_quantize", detail::block_lib().swiglu_q(detail::vp(gateUpBF16), detail::tp<uint8_t>(q), detail::tp<float>(scale),
                                                                             detail::tp<float>(amax), rows, ffnHidden, detail::vp(stream)));
}
inline void QuantizeBF16(uintptr_t xBF16, uintptr_t q, uintptr_t scale, uintptr_t amaxIn, size_t n, uintptr_t stream = 0) {
    detail::block_check("fp8_quantize_bf16", detail::block_lib().quant_bf16(detail::vp(xBF16), detail::tp<uint8_t>(q), detail::tp<float>(scale),
                                                                           detail::tp<const float>(amaxIn), n, detail::vp(stream)));
}
inline void ResidualAdd(uintptr_t x, uintptr_t yBF16, size_t n, uintptr_t stream = 0) {
    detail::block_check("fp8_residual_add", detail::block_lib().residual_add(detail::tp<float>(x), detail::vp(yBF16), n, detail::vp(stream)));
}
// Decode step: RoPE + quantise of the new token of every sequence, K and V appended to the FP8 KV cache in place
// (KVCache.Append of runs/reports/F1_HF_INFERENCE_recon.md:186-196).  Zero-initialise the struct, fill, pass.
inline void DecodeRopeAppend(const fp8_decode_append_args_t& a) {
    detail::block_check("fp8_decode_rope_append", detail::block_lib().decode_append(&a));
}

// ------------------------------------------------------------------------------- nn dispatch
// The FP8 path of goml's nn call sites — Linear.Forward (nn/linear.go:53-74), FeedForward.forwardSwiGLU
// (nn/feedforward.go:54-79), MultiHeadAttention.Forward (nn/attention.go:60-160) — on raw device buffers, and the
// Llama-style block built from them (the sequence of internal/abjexam/llama_hf_f64ref.go:94-178 with every GEMM and
// the attention in FP8).  The C++ twin of go/nn/fp8_dispatch.go, call for call.
namespace nn {

// e4m3 codes with their per-tensor scale and amax (one float each, on the device)
struct FP8Tensor { uintptr_t codes = 0, scale = 0, amax = 0; };

struct FP8Linear {   // weight [out, in], quantised once (scale = amax/448)
    int in = 0, out = 0;
    FP8Tensor w;
    // y (bf16 [M, out]) = x W^T
    void Forward(const FP8Tensor& x, int M, uintptr_t y, uintptr_t stream) const {
        FP8GEMMScaled(M, out, in, x.codes, w.codes, y, 1.0f, x.scale, w.scale, 1 /* bf16 */, stream);
    }
    // h (fp32 [M, out]) += x W^T, added in the GEMM epilogue
    void AccumulateInto(const FP8Tensor& x, int M, uintptr_t h, uintptr_t stream) const {
        FP8GEMMAccumulateF32(M, out, in, x.codes, w.codes, h, 1.0f, x.scale, w.scale, stream);
    }
};

// O = softmax(Q K^T / sqrt(hd)) V on per-tensor quantised Q, K, V [B*H, S, hd]; `scales` points at three device floats
// (Q, K, V) written by the quantiser, so nothing returns to the host in between and O is in real units.
inline void FP8Attention(FAContext& fa, uintptr_t q, uintptr_t k, uintptr_t v, uintptr_t o, uintptr_t lse, uintptr_t scales,
                         int bh, int sl, int hd, bool causal, uintptr_t stream) {
    fa_forward_args_t a{};
    a.q = detail::vp(q); a.k = detail::vp(k); a.v = detail::vp(v); a.o = detail::vp(o); a.l_out = detail::vp(lse);
    a.batch_heads = bh; a.seq_len = sl; a.head_dim = hd; a.causal = causal ? 1 : 0; a.window = 0;
    a.scale = 1.0f / std::sqrt((float)hd); a.v_descale = 1.0f;
    a.scale_q_dev = detail::tp<const float>(scales); a.scale_k_dev = detail::tp<const float>(scales + 4); a.scale_v_dev = detail::tp<const float>(scales + 8);
    a.stream = reinterpret_cast<fa_stream_t>(stream);
    fa.ForwardEx(a);
}

struct BlockBuffers {          // device buffers of one prefill pass; allocated once per shape by the caller
    uintptr_t rstd = 0;        // fp32 [T]
    FP8Tensor xq, oq, hq;      // [T, d], [T, d], [T, F]
    uintptr_t qkv = 0;         // bf16 [T, 3, H, hd]
    uintptr_t qc = 0, kc = 0, vc = 0;          // e4m3 [B*H, S, hd]
    uintptr_t qkv_scales = 0, qkv_amax = 0;    // 3 floats each
    uintptr_t o = 0;           // fp16 [B*H, S, hd]
    uintptr_t hb = 0;          // bf16 [T, F]
    uintptr_t cos = 0, sin = 0;                // fp32 [S, hd/2], from RopeTable
};

struct FP8DecoderBlock {
    int d = 0, H = 0, F = 0;
    float eps = 1e-5f;
    FP8Linear qkv, o, down;
    FP8Tensor gate_up_interleaved;   // [2*Fp, d] in the layout InterleaveGateUp produces
    uintptr_t norm1 = 0, norm2 = 0;  // fp32 [d]
    FAContext* fa = nullptr;

    // updates the fp32 residual stream h [B*S, d] in place: ten library calls, no host synchronisation
    void Forward(uintptr_t h, int B, int S, BlockBuffers& w, uintptr_t stream) const {
        const int T = B * S, hd = d / H;
        RMSNormQuantize(h, 0, 0, norm1, w.xq.codes, w.xq.scale, w.xq.amax, w.rstd, T, d, eps, stream);
        qkv.Forward(w.xq, T, w.qkv, stream);
        RopeQuantizeQKV(w.qkv, w.cos, w.sin, w.qc, w.kc, w.vc, w.qkv_scales, w.qkv_amax, B, S, H, hd, stream);
        FP8Attention(*fa, w.qc, w.kc, w.vc, w.o, 0, w.qkv_scales, B * H, S, hd, true, stream);
        PermuteQuantizeHeads(w.o, w.oq.codes, w.oq.scale, w.oq.amax, B, S, H, hd, stream);
        o.AccumulateInto(w.oq, T, h, stream);                      // h += attention projection
        RMSNormQuantize(h, 0, 0, norm2, w.xq.codes, w.xq.scale, w.xq.amax, w.rstd, T, d, eps, stream);
        FP8GEMMSwiGLU(T, F, d, w.xq.codes, gate_up_interleaved.codes, w.hb, 1.0f, w.xq.scale, gate_up_interleaved.scale, w.hq.amax, stream);
        QuantizeBF16(w.hb, w.hq.codes, w.hq.scale, w.hq.amax, (size_t)T * F, stream);
        down.AccumulateInto(w.hq, T, h, stream);                   // h += feed-forward output
    }
};

}  // namespace nn

// --------------------------------------------------------------------------- multi-GPU manager
// goml's Backend is single-device (backend/cuda/cuda..go:27,67).  The path shards with no exchange step:
// attention by contiguous batch*head ranges, the GEMM by blocks of 128-row tiles with the weight replicated.
struct Shard { long long begin, end; };

inline Shard ShardHeads(long long batchHeads, int world, int rank) {
    if (world <= 0 || rank < 0 || rank >= world) throw Error("ShardHeads: bad rank/world");
    const long long base = batchHeads / world, rem = batchHeads % world;
    const long long b = rank * base + std::min<long long>(rank, rem);
    return {b, b + base + (rank < rem ? 1 : 0)};
}
inline Shard ShardRows(long long M, int world, int rank, int tile = 128) {
    const long long tiles = (M + tile - 1) / tile;
    const Shard t = ShardHeads(tiles, world, rank);
    return {std::min(t.begin * tile, M), std::min(t.end * tile, M)};
}

// One FA context and one stream per visible device, each created with its device current.
class DeviceManager {
public:
    struct Device {
        int index;
        cudaStream_t stream;
        std::unique_ptr<FAContext> fa;
    };
    explicit DeviceManager(int maxDevices = 0) {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) throw Error("DeviceManager: no CUDA device");
        if (maxDevices > 0 && maxDevices < n) n = maxDevices;
        int prev = 0;
        cudaGetDevice(&prev);
        for (int d = 0; d < n; d++) {
            if (cudaSetDevice(d) != cudaSuccess) throw Error("DeviceManager: cudaSetDevice failed");
            Device dev{d, nullptr, nullptr};
            if (cudaStreamCreateWithFlags(&dev.stream, cudaStreamNonBlocking) != cudaSuccess) throw Error("DeviceManager: stream");
            dev.fa = FAContext::FACreate();
            devices_.push_back(std::move(dev));
        }
        cudaSetDevice(prev);
    }
    ~DeviceManager() {
        for (auto& d : devices_) {
            cudaSetDevice(d.index);
            d.fa.reset();
            if (d.stream) cudaStreamDestroy(d.stream);
        }
    }
    int Count() const { return (int)devices_.size(); }
    // Makes device i current on the calling thread (the libraries use the calling thread's device) and returns it.
    Device& Use(int i) {
        if (cudaSetDevice(devices_.at(i).index) != cudaSuccess) throw Error("DeviceManager: cudaSetDevice failed");
        return devices_[i];
    }
    void SyncAll() {
        for (auto& d : devices_) { cudaSetDevice(d.index); cudaStreamSynchronize(d.stream); }
    }

private:
    std::vector<Device> devices_;
};

}  // namespace cuda
}  // namespace goml
