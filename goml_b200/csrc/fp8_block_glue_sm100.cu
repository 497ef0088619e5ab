// fp8_block_glue_sm100.cu — libfp8block.so: RMSNorm, half-split RoPE + head permute, SwiGLU and the
// residual add of a Llama-style decoder block, each fused with the per-tensor e4m3 quantiser that
// feeds the FP8 GEMM / FP8 attention libraries.
//
// All of it is HBM-bound row-local work.  Every op runs as two kernels on the caller's stream: pass 1
// reduces the per-tensor amax of the op's fp32 result (one atomicMax per CTA), pass 2 recomputes the
// result and writes codes.  Nothing intermediate is stored, so the traffic per op is
// 2 x (input bytes) + 1 byte per output element.  Pass 2 walks the tensor backwards, so it starts on the part
// pass 1 touched last and is served from L2 (126 MB) for as much of the tensor as still sits there.  128-bit loads and stores throughout, grids sized to a multiple of the SM count.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fp8_block.h"

namespace {

constexpr int THREADS = 256;

// ---------------------------------------------------------------------------------- small helpers
// Division by a run-time constant as multiply-high + shift (numerators below 2^31): the item -> (row, column)
// decodes below would otherwise cost more instructions than the arithmetic they feed.
struct FastDiv {
    uint32_t d, mul, shr;
    FastDiv() : d(1), mul(0), shr(0) {}
    explicit FastDiv(uint32_t div) : d(div), mul(0), shr(0) {
        if (div > 1) {
            uint32_t lg = 0;
            while ((1ull << lg) < div) lg++;
            const uint32_t p = 31 + lg;
            mul = (uint32_t)(((1ull << p) + div - 1) / div);
            shr = p - 32;
        }
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : __umulhi(n, mul) >> shr; }
    __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
};
// 256-bit global loads (sm_100): one instruction per 16 bf16 / 8 fp32 values, 32-byte aligned addresses
struct U8 {
    uint32_t v[8];
};
__device__ __forceinline__ U8 ldg256(const void* p) {
    U8 r;
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
                 : "l"(p));
    return r;
}
// same through the coherent path: for buffers the kernel also writes (the residual stream updated in place)
__device__ __forceinline__ U8 ld256(const void* p) {
    U8 r;
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
                 : "l"(p)
                 : "memory");
    return r;
}
__device__ __forceinline__ void bf16x16_to_f32(const U8& r, float* f) {
#pragma unroll
    for (int k = 0; k < 8; k++) {
        f[2 * k] = __uint_as_float(r.v[k] << 16);
        f[2 * k + 1] = __uint_as_float(r.v[k] & 0xffff0000u);
    }
}
__device__ __forceinline__ void bf16x8_to_f32(const uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        f[2 * k] = __uint_as_float(w[k] << 16);
        f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
}
__device__ __forceinline__ void f16x8_to_f32(const uint4 v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 t = __half22float2(h[k]);
        f[2 * k] = t.x;
        f[2 * k + 1] = t.y;
    }
}
__device__ __forceinline__ float scale_from_amax(float amax) { return (amax > 1e-12f) ? __fdiv_rn(amax, 448.0f) : 1.0f; }

__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float inv) {
    // y * inv (one rounding), clamp, round-to-nearest-even saturating conversion: the quantiser's formula
    a = fminf(fmaxf(__fmul_rn(a, inv), -448.f), 448.f);
    b = fminf(fmaxf(__fmul_rn(b, inv), -448.f), 448.f);
    c = fminf(fmaxf(__fmul_rn(c, inv), -448.f), 448.f);
    d = fminf(fmaxf(__fmul_rn(d, inv), -448.f), 448.f);
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}
__device__ __forceinline__ uint4 quant16(const float* y, float inv) {
    return make_uint4(quant4(y[0], y[1], y[2], y[3], inv), quant4(y[4], y[5], y[6], y[7], inv),
                      quant4(y[8], y[9], y[10], y[11], inv), quant4(y[12], y[13], y[14], y[15], inv));
}
__device__ __forceinline__ float absmax16(const float* y, float m) {
#pragma unroll
    for (int i = 0; i < 16; i++) m = fmaxf(m, fabsf(y[i]));  // NaN never wins
    return m;
}

__device__ __forceinline__ float block_max(float m, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();  // sh may still be read from a previous call
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
    __syncthreads();
    m = sh[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; w++) m = fmaxf(m, sh[w]);
    return m;
}
__device__ __forceinline__ float block_sum(float s, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    s = sh[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; w++) s += sh[w];  // fixed order: the same in every CTA
    return s;
}
// non-negative floats order like their bit patterns
__device__ __forceinline__ void atomic_amax(float* amax, float m) { atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m)); }

int grid_for(size_t items) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t blocks = (items + THREADS - 1) / THREADS;
    const size_t cap = (size_t)sms * 8;  // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}
bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }
bool misaligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) != 0; }  // operands of 256-bit loads

// ---------------------------------------------------------------------------------- RoPE table
__global__ void rope_table_kernel(float* cos_out, float* sin_out, int seq_len, int half, double theta, double hd) {
    const int n = seq_len * half;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
        const int s = idx / half, i = idx % half;
        const double ang = (double)s * pow(theta, -2.0 * (double)i / hd);
        double sv, cv;
        sincos(ang, &sv, &cv);
        cos_out[idx] = (float)cv;
        sin_out[idx] = (float)sv;
    }
}

// ---------------------------------------------------------------------------------- RMSNorm (+ residual) + quantise
// h = x (+ residual) for 4 consecutive elements
__device__ __forceinline__ float4 load_h4(const float* x, const uint16_t* res, size_t off) {
    float4 h = *reinterpret_cast<const float4*>(x + off);
    if (res) {
        const uint2 r = *reinterpret_cast<const uint2*>(res + off);
        h.x += __uint_as_float(r.x << 16);
        h.y += __uint_as_float(r.x & 0xffff0000u);
        h.z += __uint_as_float(r.y << 16);
        h.w += __uint_as_float(r.y & 0xffff0000u);
    }
    return h;
}

// The normalised value is evaluated as y = (h * gamma) * rstd, each product rounded to fp32.  Multiplying by the
// positive row constant rstd is monotonic even after rounding, so max_i |y_i| of a row is exactly
// fl(max_i |fl(h_i * gamma_i)| * rstd): pass 1 needs ONE sweep over the row (sum of squares and that maximum
// together) and one block-wide reduction, instead of a second sweep that waits for rstd.
__device__ __forceinline__ void block_sum_max(float& s, float& m, float* sh) {  // sh[2 * THREADS / 32]
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    __syncthreads();  // sh may still be read from the previous row
    if ((threadIdx.x & 31) == 0) {
        sh[threadIdx.x >> 5] = s;
        sh[THREADS / 32 + (threadIdx.x >> 5)] = m;
    }
    __syncthreads();
    s = sh[0];
    m = sh[THREADS / 32];
#pragma unroll
    for (int w = 1; w < THREADS / 32; w++) {  // fixed order: the same in every CTA
        s += sh[w];
        m = fmaxf(m, sh[THREADS / 32 + w]);
    }
}

// pass 1, any hidden (multiple of 16): one CTA per row (grid-stride): h_out, rstd per row, amax
__global__ void __launch_bounds__(THREADS) rms_stats_kernel(const float* __restrict__ x, const uint16_t* __restrict__ res,
                                                            float* h_out, const float* __restrict__ gamma,
                                                            float* __restrict__ rstd_ws, float* amax, int rows, int hidden,
                                                            float eps) {
    __shared__ float sh[2 * THREADS / 32];
    float run_max = 0.f;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * hidden;
        float ss = 0.f, m1 = 0.f;
        for (int c = threadIdx.x * 4; c < hidden; c += THREADS * 4) {
            const float4 h = load_h4(x, res, base + c);
            if (res && h_out) *reinterpret_cast<float4*>(h_out + base + c) = h;
            const float4 g = *reinterpret_cast<const float4*>(gamma + c);
            ss = fmaf(h.x, h.x, ss);
            ss = fmaf(h.y, h.y, ss);
            ss = fmaf(h.z, h.z, ss);
            ss = fmaf(h.w, h.w, ss);
            m1 = fmaxf(fmaxf(m1, fmaxf(fabsf(__fmul_rn(h.x, g.x)), fabsf(__fmul_rn(h.y, g.y)))),
                       fmaxf(fabsf(__fmul_rn(h.z, g.z)), fabsf(__fmul_rn(h.w, g.w))));
        }
        block_sum_max(ss, m1, sh);
        const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps));
        if (threadIdx.x == 0) rstd_ws[row] = rstd;
        run_max = fmaxf(run_max, __fmul_rn(m1, rstd));
    }
    if (threadIdx.x == 0) atomic_amax(amax, run_max);
}

// pass 1 for hidden = N * 2048 (N = 1, 2, 4): the row lives in registers (N 256-bit loads per thread) and the
// next row's loads are issued before this row's reductions, so the two block-wide reductions per row no longer
// drain the memory pipeline.
__device__ __forceinline__ void st256(void* p, const U8& r) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.v[0]), "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]),
                 "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7])
                 : "memory");
}
template <int N, bool HAS_RES>
struct RowRegs {
    U8 x[N];
    uint4 r[HAS_RES ? N : 1];
};
template <int N, bool HAS_RES>
__device__ __forceinline__ void load_row(RowRegs<N, HAS_RES>& t, const float* x, const uint16_t* res, size_t base) {
#pragma unroll
    for (int k = 0; k < N; k++) {
        const size_t off = base + (size_t)k * (THREADS * 8) + threadIdx.x * 8;
        t.x[k] = ld256(x + off);
        if (HAS_RES) t.r[k] = __ldg(reinterpret_cast<const uint4*>(res + off));
    }
}
template <int N, bool HAS_RES>
__global__ void __launch_bounds__(THREADS) rms_stats_regs_kernel(const float* __restrict__ x, const uint16_t* __restrict__ res, float* h_out,
                                                                 const float* __restrict__ gamma, float* __restrict__ rstd_ws, float* amax,
                                                                 int rows, float eps) {
    constexpr int hidden = N * THREADS * 8;
    __shared__ float sh[2 * THREADS / 32];
    float run_max = 0.f;
    U8 g[N];
#pragma unroll
    for (int k = 0; k < N; k++) g[k] = ldg256(gamma + k * (THREADS * 8) + threadIdx.x * 8);
    RowRegs<N, HAS_RES> cur, nxt;
    int row = blockIdx.x;
    if (row < rows) load_row<N, HAS_RES>(cur, x, res, (size_t)row * hidden);
    for (; row < rows; row += gridDim.x) {
        const int next = row + gridDim.x;
        if (next < rows) load_row<N, HAS_RES>(nxt, x, res, (size_t)next * hidden);
        float ss = 0.f, m1 = 0.f;
#pragma unroll
        for (int k = 0; k < N; k++) {
            float rf[8];
            if (HAS_RES) bf16x8_to_f32(cur.r[k], rf);
            U8 o;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float h = __uint_as_float(cur.x[k].v[i]);
                if (HAS_RES) h += rf[i];
                o.v[i] = __float_as_uint(h);
                ss = fmaf(h, h, ss);
                m1 = fmaxf(m1, fabsf(__fmul_rn(h, __uint_as_float(g[k].v[i]))));
            }
            if (HAS_RES && h_out) st256(h_out + (size_t)row * hidden + (size_t)k * (THREADS * 8) + threadIdx.x * 8, o);
        }
        block_sum_max(ss, m1, sh);
        const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps));
        if (threadIdx.x == 0) rstd_ws[row] = rstd;
        run_max = fmaxf(run_max, __fmul_rn(m1, rstd));
        if (next < rows) cur = nxt;
    }
    if (threadIdx.x == 0) atomic_amax(amax, run_max);
}

// pass 2: 16 elements per thread per step
__global__ void __launch_bounds__(THREADS) rms_quant_kernel(const float* __restrict__ h_src, const uint16_t* __restrict__ res,
                                                            const float* __restrict__ gamma, const float* __restrict__ rstd_ws,
                                                            const float* __restrict__ amax_ptr, float* scale_out,
                                                            uint8_t* __restrict__ q, uint32_t items, int hidden,
                                                            const FastDiv per_row) {
    const float scale = scale_from_amax(*amax_ptr);
    const float inv = __fdiv_rn(1.0f, scale);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    // two items per step, all loads issued before the first use: twice the bytes in flight per thread
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < items; it += 2 * stride) {
        uint32_t row[2], c[2];
        bool live[2];
        U8 hv[2][2], gv[2][2];
        float rstd[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t i = it + u * stride;
            live[u] = i < items;
            per_row.divmod(items - 1 - (live[u] ? i : it), row[u], c[u]);  // backwards: the rows pass 1 finished with are still in L2
            c[u] *= 16;
            const size_t off = (size_t)row[u] * hidden + c[u];
            hv[u][0] = ldg256(h_src + off);
            hv[u][1] = ldg256(h_src + off + 8);
            gv[u][0] = ldg256(gamma + c[u]);
            gv[u][1] = ldg256(gamma + c[u] + 8);
            rstd[u] = rstd_ws[row[u]];
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            if (!live[u]) continue;
            const size_t off = (size_t)row[u] * hidden + c[u];
            float y[16];
#pragma unroll
            for (int v = 0; v < 16; v++) {
                float h = __uint_as_float(hv[u][v >> 3].v[v & 7]);
                if (res) {
                    const uint16_t r = res[off + v];
                    h += __uint_as_float((uint32_t)r << 16);
                }
                y[v] = __fmul_rn(__fmul_rn(h, __uint_as_float(gv[u][v >> 3].v[v & 7])), rstd[u]);
            }
            *reinterpret_cast<uint4*>(q + off) = quant16(y, inv);
        }
    }
}

// ---------------------------------------------------------------------------------- RoPE + permute + quantise of Q, K, V
// One item = 32 elements of one (token, tensor, head): for Q and K the 16 rotation pairs
// (i, i + hd/2), i in [16c, 16c+16); for V the elements [32c, 32c+32).
struct QkvItem {
    int which, b, s, h, c;
};
struct QkvDivs {
    FastDiv cph, heads, three, seq;
};
__device__ __forceinline__ QkvItem decode_qkv(uint32_t it, const QkvDivs& dv) {
    QkvItem r;
    uint32_t q, m;
    dv.cph.divmod(it, q, m);
    r.c = (int)m;
    dv.heads.divmod(q, q, m);
    r.h = (int)m;
    dv.three.divmod(q, q, m);
    r.which = (int)m;
    dv.seq.divmod(q, q, m);
    r.s = (int)m;
    r.b = (int)q;
    return r;
}
// y[0..15] = first-half results (or V elements 0..15), y[16..31] = second-half results (or V 16..31)
__device__ __forceinline__ void qkv_values(const uint16_t* __restrict__ qkv, const float* __restrict__ cos_tab,
                                           const float* __restrict__ sin_tab, const QkvItem& t, int seq_len, int heads, int hd,
                                           float* y) {
    const int half = hd / 2;
    const size_t row = ((size_t)t.b * seq_len + t.s) * 3 * heads * hd + ((size_t)t.which * heads + t.h) * hd;
    if (t.which == 2) {
        const uint4* src = reinterpret_cast<const uint4*>(qkv + row + 32 * t.c);
#pragma unroll
        for (int v = 0; v < 4; v++) bf16x8_to_f32(__ldg(src + v), y + 8 * v);
        return;
    }
    float x0[16], x1[16];
    const uint4* s0 = reinterpret_cast<const uint4*>(qkv + row + 16 * t.c);
    const uint4* s1 = reinterpret_cast<const uint4*>(qkv + row + half + 16 * t.c);
    bf16x8_to_f32(__ldg(s0), x0);
    bf16x8_to_f32(__ldg(s0 + 1), x0 + 8);
    bf16x8_to_f32(__ldg(s1), x1);
    bf16x8_to_f32(__ldg(s1 + 1), x1 + 8);
    const float4* ct = reinterpret_cast<const float4*>(cos_tab + (size_t)t.s * half + 16 * t.c);
    const float4* st = reinterpret_cast<const float4*>(sin_tab + (size_t)t.s * half + 16 * t.c);
#pragma unroll
    for (int v = 0; v < 4; v++) {
        const float4 c4 = __ldg(ct + v), s4 = __ldg(st + v);
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int i = 4 * v + e;
            // x0 c - x1 s ; x0 s + x1 c  (each product rounded, then one add: no contraction)
            y[i] = __fsub_rn(__fmul_rn(x0[i], cc[e]), __fmul_rn(x1[i], ss[e]));
            y[16 + i] = __fadd_rn(__fmul_rn(x0[i], ss[e]), __fmul_rn(x1[i], cc[e]));
        }
    }
}

__global__ void __launch_bounds__(THREADS) qkv_amax_kernel(const uint16_t* __restrict__ qkv, const float* __restrict__ cos_tab,
                                                           const float* __restrict__ sin_tab, float* amaxes, uint32_t items,
                                                           int seq_len, int heads, int hd, const QkvDivs dv) {
    __shared__ float sh[THREADS / 32];
    float m[3] = {0.f, 0.f, 0.f};
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < items; it += gridDim.x * blockDim.x) {
        const QkvItem t = decode_qkv(it, dv);
        float y[32];
        qkv_values(qkv, cos_tab, sin_tab, t, seq_len, heads, hd, y);
        const float a = absmax16(y + 16, absmax16(y, 0.f));
        if (t.which == 0) m[0] = fmaxf(m[0], a);
        else if (t.which == 1) m[1] = fmaxf(m[1], a);
        else m[2] = fmaxf(m[2], a);
    }
#pragma unroll
    for (int w = 0; w < 3; w++) {
        const float r = block_max(m[w], sh);
        if (threadIdx.x == 0) atomic_amax(amaxes + w, r);
    }
}

__global__ void __launch_bounds__(THREADS) qkv_quant_kernel(const uint16_t* __restrict__ qkv, const float* __restrict__ cos_tab,
                                                            const float* __restrict__ sin_tab, const float* __restrict__ amaxes,
                                                            float* scales, uint8_t* __restrict__ q_out, uint8_t* __restrict__ k_out,
                                                            uint8_t* __restrict__ v_out, uint32_t items, int seq_len, int heads, int hd,
                                                            const QkvDivs dv) {
    float inv[3];
#pragma unroll
    for (int w = 0; w < 3; w++) {
        const float sc = scale_from_amax(amaxes[w]);
        inv[w] = __fdiv_rn(1.0f, sc);
        if (blockIdx.x == 0 && threadIdx.x == 0) scales[w] = sc;
    }
    const int half = hd / 2;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < items; it += gridDim.x * blockDim.x) {
        const QkvItem t = decode_qkv(items - 1 - it, dv);  // backwards: see the file header
        float y[32];
        qkv_values(qkv, cos_tab, sin_tab, t, seq_len, heads, hd, y);
        uint8_t* dst = (t.which == 0 ? q_out : t.which == 1 ? k_out : v_out) + (((size_t)t.b * heads + t.h) * seq_len + t.s) * hd;
        const float iv = t.which == 0 ? inv[0] : t.which == 1 ? inv[1] : inv[2];
        if (t.which == 2) {
            *reinterpret_cast<uint4*>(dst + 32 * t.c) = quant16(y, iv);
            *reinterpret_cast<uint4*>(dst + 32 * t.c + 16) = quant16(y + 16, iv);
        } else {
            *reinterpret_cast<uint4*>(dst + 16 * t.c) = quant16(y, iv);
            *reinterpret_cast<uint4*>(dst + half + 16 * t.c) = quant16(y + 16, iv);
        }
    }
}

// ---------------------------------------------------------------------------------- decode step: RoPE + quantise + cache append
// One item = 32 elements of one (sequence, head slot): slots [0, Hq) are query heads, [Hq, Hq+Hkv) key heads,
// [Hq+Hkv, Hq+2Hkv) value heads of the new token's projection row.  Q and K items are 16 rotation pairs as above.
struct DecAppend {
    const uint16_t* qkv;
    const float* cos_tab;
    const float* sin_tab;
    const int* positions;
    uint8_t* q_out;
    float* q_scale;
    float* q_amax;
    uint8_t* k_cache;
    uint8_t* v_cache;
    const float* k_scale;
    const float* v_scale;
    int* seq_lens_out;
    const int* block_table;
    int batch, hq, hkv, hd, s_max, table_rows, page_size, max_pages, num_pages;
    uint32_t items;
    FastDiv cph, slots;
};
// position of sequence b's new token, or -1 when it cannot be placed (an inactive slot, a full cache, no RoPE row)
__device__ __forceinline__ int dec_position(const DecAppend& a, int b) {
    const int pos = __ldg(a.positions + b);
    const int cap = a.block_table ? a.page_size * a.max_pages : a.s_max;
    return (pos >= 0 && pos < cap && pos < a.table_rows) ? pos : -1;
}
__device__ __forceinline__ void dec_values(const DecAppend& a, int b, int slot, int c, int pos, float* y) {
    const int half = a.hd / 2;
    const size_t row = ((size_t)b * (a.hq + 2 * a.hkv) + slot) * a.hd;
    if (slot >= a.hq + a.hkv) {
        const uint4* src = reinterpret_cast<const uint4*>(a.qkv + row + 32 * c);
#pragma unroll
        for (int v = 0; v < 4; v++) bf16x8_to_f32(__ldg(src + v), y + 8 * v);
        return;
    }
    float x0[16], x1[16];
    const uint4* s0 = reinterpret_cast<const uint4*>(a.qkv + row + 16 * c);
    const uint4* s1 = reinterpret_cast<const uint4*>(a.qkv + row + half + 16 * c);
    bf16x8_to_f32(__ldg(s0), x0);
    bf16x8_to_f32(__ldg(s0 + 1), x0 + 8);
    bf16x8_to_f32(__ldg(s1), x1);
    bf16x8_to_f32(__ldg(s1 + 1), x1 + 8);
    const float* ct = a.cos_tab + (size_t)pos * half + 16 * c;
    const float* st = a.sin_tab + (size_t)pos * half + 16 * c;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const float cc = __ldg(ct + i), ss = __ldg(st + i);
        y[i] = __fsub_rn(__fmul_rn(x0[i], cc), __fmul_rn(x1[i], ss));
        y[16 + i] = __fadd_rn(__fmul_rn(x0[i], ss), __fmul_rn(x1[i], cc));
    }
}
__global__ void __launch_bounds__(THREADS) dec_q_amax_kernel(const DecAppend a) {
    __shared__ float sh[THREADS / 32];
    float m = 0.f;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < a.items; it += gridDim.x * blockDim.x) {
        uint32_t q, c, b, slot;
        a.cph.divmod(it, q, c);
        a.slots.divmod(q, b, slot);
        if ((int)slot >= a.hq) continue;
        const int pos = dec_position(a, (int)b);
        if (pos < 0) continue;
        float y[32];
        dec_values(a, (int)b, (int)slot, (int)c, pos, y);
        m = absmax16(y + 16, absmax16(y, m));
    }
    m = block_max(m, sh);
    if (threadIdx.x == 0) atomic_amax(a.q_amax, m);
}
__global__ void __launch_bounds__(THREADS) dec_append_kernel(const DecAppend a) {
    const float q_sc = scale_from_amax(*a.q_amax);
    const float inv_q = __fdiv_rn(1.0f, q_sc);
    const float inv_k = __fdiv_rn(1.0f, __ldg(a.k_scale)), inv_v = __fdiv_rn(1.0f, __ldg(a.v_scale));
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.q_scale = q_sc;
    const int half = a.hd / 2;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < a.items; it += gridDim.x * blockDim.x) {
        uint32_t q, c, b, slot;
        a.cph.divmod(it, q, c);
        a.slots.divmod(q, b, slot);
        const int pos = dec_position(a, (int)b);
        if (slot == 0 && c == 0 && a.seq_lens_out) {
            // an inactive slot keeps its length: 0 for a negative position, the capacity for a full cache
            const int raw = __ldg(a.positions + b);
            const int cap = a.block_table ? a.page_size * a.max_pages : a.s_max;
            a.seq_lens_out[b] = pos >= 0 ? pos + 1 : (raw < 0 ? 0 : min(raw, cap));
        }
        if ((int)slot < a.hq) {
            uint8_t* dst = a.q_out + ((size_t)b * a.hq + slot) * a.hd;
            if (pos < 0) {  // an inactive sequence: zero codes, nothing appended
                *reinterpret_cast<uint4*>(dst + 16 * c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(dst + half + 16 * c) = make_uint4(0, 0, 0, 0);
                continue;
            }
            float y[32];
            dec_values(a, (int)b, (int)slot, (int)c, pos, y);
            *reinterpret_cast<uint4*>(dst + 16 * c) = quant16(y, inv_q);
            *reinterpret_cast<uint4*>(dst + half + 16 * c) = quant16(y + 16, inv_q);
            continue;
        }
        if (pos < 0) continue;
        const bool is_v = (int)slot >= a.hq + a.hkv;
        const int h = (int)slot - a.hq - (is_v ? a.hkv : 0);
        size_t key_row;   // index of this (sequence, kv head, position) among the cache's rows of hd codes
        if (a.block_table) {
            const int pg = pos / a.page_size;
            const int page = __ldg(a.block_table + (size_t)b * a.max_pages + pg);
            if (page < 0 || page >= a.num_pages) continue;   // no page behind this position: nothing is written
            key_row = ((size_t)page * a.hkv + h) * a.page_size + (pos - pg * a.page_size);
        } else {
            key_row = ((size_t)b * a.hkv + h) * a.s_max + pos;
        }
        float y[32];
        dec_values(a, (int)b, (int)slot, (int)c, pos, y);
        uint8_t* dst = (is_v ? a.v_cache : a.k_cache) + key_row * a.hd;
        if (is_v) {
            *reinterpret_cast<uint4*>(dst + 32 * c) = quant16(y, inv_v);
            *reinterpret_cast<uint4*>(dst + 32 * c + 16) = quant16(y + 16, inv_v);
        } else {
            *reinterpret_cast<uint4*>(dst + 16 * c) = quant16(y, inv_k);
            *reinterpret_cast<uint4*>(dst + half + 16 * c) = quant16(y + 16, inv_k);
        }
    }
}

// ---------------------------------------------------------------------------------- attention output: permute + quantise
// item = 16 consecutive elements of one (token, head); out index order so that stores are contiguous
struct ODivs {
    FastDiv cph, heads, seq;
};
__device__ __forceinline__ size_t o_src_offset(uint32_t it, int seq_len, int heads, int hd, const ODivs& dv) {
    uint32_t q, c, h, s;
    dv.cph.divmod(it, q, c);
    dv.heads.divmod(q, q, h);
    dv.seq.divmod(q, q, s);  // q = batch index
    return (((size_t)q * heads + h) * seq_len + s) * hd + 16 * c;
}
__global__ void __launch_bounds__(THREADS) o_amax_kernel(const uint16_t* __restrict__ o, float* amax, size_t n16) {
    __shared__ float sh[THREADS / 32];
    float m = 0.f;
    const uint4* src = reinterpret_cast<const uint4*>(o);
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < n16; it += (size_t)gridDim.x * blockDim.x) {
        float y[16];
        f16x8_to_f32(__ldg(src + 2 * it), y);
        f16x8_to_f32(__ldg(src + 2 * it + 1), y + 8);
        m = absmax16(y, m);
    }
    m = block_max(m, sh);
    if (threadIdx.x == 0) atomic_amax(amax, m);
}
__global__ void __launch_bounds__(THREADS) o_quant_kernel(const uint16_t* __restrict__ o, const float* __restrict__ amax_ptr,
                                                          float* scale_out, uint8_t* __restrict__ q, uint32_t n16, int seq_len,
                                                          int heads, int hd, const ODivs dv) {
    const float scale = scale_from_amax(*amax_ptr);
    const float inv = __fdiv_rn(1.0f, scale);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < n16; it += gridDim.x * blockDim.x) {
        const uint32_t rit = n16 - 1 - it;   // destination order (token-major), walked backwards
        const uint4* sp = reinterpret_cast<const uint4*>(o + o_src_offset(rit, seq_len, heads, hd, dv));
        float y[16];
        f16x8_to_f32(__ldg(sp), y);
        f16x8_to_f32(__ldg(sp + 1), y + 8);
        *reinterpret_cast<uint4*>(q + (size_t)rit * 16) = quant16(y, inv);
    }
}

// ---------------------------------------------------------------------------------- SwiGLU + quantise
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void swiglu16(const U8& gv, const U8& uv, float* y) {
    float g[16], u[16];
    bf16x16_to_f32(gv, g);
    bf16x16_to_f32(uv, u);
#pragma unroll
    for (int i = 0; i < 16; i++)  // g / (1 + e^-g) * u with the hardware exponential and reciprocal (a few fp32 ulp)
        y[i] = __fmul_rn(__fmul_rn(g[i], rcp_approx(__fadd_rn(1.0f, __expf(-g[i])))), u[i]);
}
__global__ void __launch_bounds__(THREADS) swiglu_amax_kernel(const uint16_t* __restrict__ gu, float* amax, uint32_t items, int F,
                                                              const FastDiv per_row) {
    __shared__ float sh[THREADS / 32];
    float m = 0.f;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < items; it += 2 * stride) {  // two items per step, loads first
        U8 gv[2], uv[2];
        bool live[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t i = it + u * stride;
            live[u] = i < items;
            uint32_t row, c;
            per_row.divmod(live[u] ? i : it, row, c);
            const uint16_t* gp = gu + (size_t)row * 2 * F + c * 16;
            gv[u] = ldg256(gp);
            uv[u] = ldg256(gp + F);
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            float y[16];
            swiglu16(gv[u], uv[u], y);
            if (live[u]) m = absmax16(y, m);
        }
    }
    m = block_max(m, sh);
    if (threadIdx.x == 0) atomic_amax(amax, m);
}
__global__ void __launch_bounds__(THREADS) swiglu_quant_kernel(const uint16_t* __restrict__ gu, const float* __restrict__ amax_ptr,
                                                               float* scale_out, uint8_t* __restrict__ q, uint32_t items, int F,
                                                               const FastDiv per_row) {
    const float scale = scale_from_amax(*amax_ptr);
    const float inv = __fdiv_rn(1.0f, scale);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < items; it += 2 * stride) {  // two items per step, loads first
        U8 gv[2], uv[2];
        bool live[2];
        size_t dst[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t i = it + u * stride;
            live[u] = i < items;
            uint32_t row, c;
            per_row.divmod(items - 1 - (live[u] ? i : it), row, c);  // backwards: see the file header
            const uint16_t* gp = gu + (size_t)row * 2 * F + c * 16;
            gv[u] = ldg256(gp);
            uv[u] = ldg256(gp + F);
            dst[u] = (size_t)row * F + c * 16;
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            float y[16];
            swiglu16(gv[u], uv[u], y);
            if (live[u]) *reinterpret_cast<uint4*>(q + dst[u]) = quant16(y, inv);
        }
    }
}

// ---------------------------------------------------------------------------------- quantise bf16 with a known amax
// single pass: the producer (the SwiGLU GEMM epilogue) already reduced max|x|
__global__ void __launch_bounds__(THREADS) quant_bf16_kernel(const uint16_t* __restrict__ x, const float* __restrict__ amax_ptr,
                                                             float* scale_out, uint8_t* __restrict__ q, size_t n16) {
    const float scale = scale_from_amax(*amax_ptr);
    const float inv = __fdiv_rn(1.0f, scale);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < n16; it += 2 * stride) {  // two items per step, loads first
        const bool second = it + stride < n16;
        const U8 a = ldg256(x + it * 16);
        const U8 b = ldg256(x + (second ? it + stride : it) * 16);
        float y[16];
        bf16x16_to_f32(a, y);
        *reinterpret_cast<uint4*>(q + it * 16) = quant16(y, inv);
        if (second) {
            bf16x16_to_f32(b, y);
            *reinterpret_cast<uint4*>(q + (it + stride) * 16) = quant16(y, inv);
        }
    }
}

// ---------------------------------------------------------------------------------- residual add
__global__ void __launch_bounds__(THREADS) residual_add_kernel(float* __restrict__ x, const uint16_t* __restrict__ y, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        float f[8];
        bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(y) + i), f);
        float4* xp = reinterpret_cast<float4*>(x) + 2 * i;
        float4 a = xp[0], b = xp[1];
        a.x += f[0]; a.y += f[1]; a.z += f[2]; a.w += f[3];
        b.x += f[4]; b.y += f[5]; b.z += f[6]; b.w += f[7];
        xp[0] = a;
        xp[1] = b;
    }
}

}  // namespace

extern "C" {

int fp8_rope_table(float* cos_out, float* sin_out, int seq_len, int head_dim, float theta, void* stream) {
    if (!cos_out || !sin_out || seq_len <= 0 || head_dim <= 0 || (head_dim & 1) || !(theta > 0.f)) return (int)cudaErrorInvalidValue;
    const int half = head_dim / 2;
    rope_table_kernel<<<grid_for((size_t)seq_len * half), THREADS, 0, (cudaStream_t)stream>>>(cos_out, sin_out, seq_len, half,
                                                                                             (double)theta, (double)head_dim);
    return (int)cudaGetLastError();
}

int fp8_rmsnorm_quantize(const float* x, const void* residual_bf16, float* h_out, const float* gamma, uint8_t* q,
                         float* scale_out, float* amax_out, float* rstd_ws, int rows, int hidden, float eps, void* stream) {
    if (!x || !gamma || !q || !scale_out || !amax_out || !rstd_ws) return (int)cudaErrorInvalidValue;
    if (rows < 0 || hidden <= 0 || (hidden % 16) != 0) return (int)cudaErrorInvalidValue;
    if (misaligned32(x) || misaligned(residual_bf16) || misaligned32(h_out) || misaligned32(gamma) || misaligned(q)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const uint16_t* res = reinterpret_cast<const uint16_t*>(residual_bf16);
    if (rows > 0) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int grid = rows < sms * 8 ? rows : sms * 8;
#define RMS_STATS_REGS(N)                                                                                               \
    (res ? rms_stats_regs_kernel<N, true><<<grid, THREADS, 0, s>>>(x, res, h_out, gamma, rstd_ws, amax_out, rows, eps) \
         : rms_stats_regs_kernel<N, false><<<grid, THREADS, 0, s>>>(x, res, h_out, gamma, rstd_ws, amax_out, rows, eps))
        if (hidden == 2048) RMS_STATS_REGS(1);
        else if (hidden == 4096) RMS_STATS_REGS(2);
        else if (hidden == 8192) RMS_STATS_REGS(4);
        else rms_stats_kernel<<<grid, THREADS, 0, s>>>(x, res, h_out, gamma, rstd_ws, amax_out, rows, hidden, eps);
#undef RMS_STATS_REGS
    }
    // pass 2 reads the updated stream where pass 1 stored it
    const bool from_h = res && h_out;
    const size_t items = (size_t)rows * (hidden / 16);
    if (items >= (1ull << 31)) return (int)cudaErrorInvalidValue;
    rms_quant_kernel<<<grid_for(items), THREADS, 0, s>>>(from_h ? h_out : x, from_h ? nullptr : res, gamma, rstd_ws, amax_out, scale_out, q,
                                                         (uint32_t)items, hidden, FastDiv(hidden / 16));
    return (int)cudaGetLastError();
}

int fp8_rope_quantize_qkv(const void* qkv_bf16, const float* cos_tab, const float* sin_tab, uint8_t* q_out, uint8_t* k_out,
                          uint8_t* v_out, float* scales, float* amaxes, int batch, int seq_len, int heads, int head_dim,
                          void* stream) {
    if (!qkv_bf16 || !cos_tab || !sin_tab || !q_out || !k_out || !v_out || !scales || !amaxes) return (int)cudaErrorInvalidValue;
    if (batch < 0 || seq_len <= 0 || heads <= 0 || (head_dim != 64 && head_dim != 128)) return (int)cudaErrorInvalidValue;
    if (misaligned(qkv_bf16) || misaligned(cos_tab) || misaligned(sin_tab) || misaligned(q_out) || misaligned(k_out) || misaligned(v_out))
        return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(amaxes, 0, 3 * sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const size_t items = (size_t)batch * seq_len * 3 * heads * (head_dim / 32);
    if (items >= (1ull << 31)) return (int)cudaErrorInvalidValue;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(qkv_bf16);
    QkvDivs dv;
    dv.cph = FastDiv(head_dim / 32);
    dv.heads = FastDiv(heads);
    dv.three = FastDiv(3);
    dv.seq = FastDiv(seq_len);
    if (items > 0)
        qkv_amax_kernel<<<grid_for(items), THREADS, 0, s>>>(src, cos_tab, sin_tab, amaxes, (uint32_t)items, seq_len, heads, head_dim, dv);
    qkv_quant_kernel<<<grid_for(items), THREADS, 0, s>>>(src, cos_tab, sin_tab, amaxes, scales, q_out, k_out, v_out, (uint32_t)items, seq_len,
                                                         heads, head_dim, dv);
    return (int)cudaGetLastError();
}

int fp8_decode_rope_append(const fp8_decode_append_args_t* g) {
    if (!g || !g->qkv_bf16 || !g->cos_tab || !g->sin_tab || !g->positions || !g->q_out || !g->q_scale_out || !g->q_amax_out ||
        !g->k_cache || !g->v_cache || !g->k_scale || !g->v_scale)
        return (int)cudaErrorInvalidValue;
    if (g->batch < 0 || g->q_heads <= 0 || g->kv_heads <= 0 || (g->head_dim != 64 && g->head_dim != 128) || g->rope_rows <= 0)
        return (int)cudaErrorInvalidValue;
    if (g->block_table) {
        if (g->page_size <= 0 || g->max_pages_per_seq <= 0 || g->num_pages <= 0 ||
            (long long)g->page_size * g->max_pages_per_seq > 0x7fffffffLL)
            return (int)cudaErrorInvalidValue;
    } else if (g->s_max <= 0) {
        return (int)cudaErrorInvalidValue;
    }
    if (misaligned(g->qkv_bf16) || misaligned(g->q_out) || misaligned(g->k_cache) || misaligned(g->v_cache)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)g->stream;
    cudaError_t e = cudaMemsetAsync(g->q_amax_out, 0, sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const int slots = g->q_heads + 2 * g->kv_heads;
    const size_t items = (size_t)g->batch * slots * (g->head_dim / 32);
    if (items >= (1ull << 31)) return (int)cudaErrorInvalidValue;
    DecAppend a;
    a.qkv = reinterpret_cast<const uint16_t*>(g->qkv_bf16);
    a.cos_tab = g->cos_tab; a.sin_tab = g->sin_tab; a.positions = g->positions;
    a.q_out = g->q_out; a.q_scale = g->q_scale_out; a.q_amax = g->q_amax_out;
    a.k_cache = g->k_cache; a.v_cache = g->v_cache; a.k_scale = g->k_scale; a.v_scale = g->v_scale;
    a.seq_lens_out = g->seq_lens_out; a.block_table = g->block_table;
    a.batch = g->batch; a.hq = g->q_heads; a.hkv = g->kv_heads; a.hd = g->head_dim; a.s_max = g->s_max;
    a.table_rows = g->rope_rows; a.page_size = g->page_size; a.max_pages = g->max_pages_per_seq; a.num_pages = g->num_pages;
    a.items = (uint32_t)items;
    a.cph = FastDiv(g->head_dim / 32);
    a.slots = FastDiv(slots);
    if (items > 0) dec_q_amax_kernel<<<grid_for(items), THREADS, 0, s>>>(a);
    dec_append_kernel<<<grid_for(items), THREADS, 0, s>>>(a);
    return (int)cudaGetLastError();
}

int fp8_permute_quantize_heads(const void* o_fp16, uint8_t* q, float* scale_out, float* amax_out, int batch, int seq_len,
                               int heads, int head_dim, void* stream) {
    if (!o_fp16 || !q || !scale_out || !amax_out) return (int)cudaErrorInvalidValue;
    if (batch < 0 || seq_len <= 0 || heads <= 0 || head_dim <= 0 || (head_dim % 16) != 0) return (int)cudaErrorInvalidValue;
    if (misaligned(o_fp16) || misaligned(q)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const size_t n16 = (size_t)batch * seq_len * heads * (head_dim / 16);
    if (n16 >= (1ull << 31)) return (int)cudaErrorInvalidValue;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(o_fp16);
    ODivs dv;
    dv.cph = FastDiv(head_dim / 16);
    dv.heads = FastDiv(heads);
    dv.seq = FastDiv(seq_len);
    if (n16 > 0) o_amax_kernel<<<grid_for(n16), THREADS, 0, s>>>(src, amax_out, n16);
    o_quant_kernel<<<grid_for(n16), THREADS, 0, s>>>(src, amax_out, scale_out, q, (uint32_t)n16, seq_len, heads, head_dim, dv);
    return (int)cudaGetLastError();
}

int fp8_swiglu_quantize(const void* gate_up_bf16, uint8_t* q, float* scale_out, float* amax_out, int rows, int ffn_hidden,
                        void* stream) {
    if (!gate_up_bf16 || !q || !scale_out || !amax_out) return (int)cudaErrorInvalidValue;
    if (rows < 0 || ffn_hidden <= 0 || (ffn_hidden % 16) != 0) return (int)cudaErrorInvalidValue;
    if (misaligned32(gate_up_bf16) || misaligned(q)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(gate_up_bf16);
    const size_t items = (size_t)rows * (ffn_hidden / 16);
    if (items >= (1ull << 31)) return (int)cudaErrorInvalidValue;
    const FastDiv per_row(ffn_hidden / 16);
    if (items > 0) swiglu_amax_kernel<<<grid_for(items), THREADS, 0, s>>>(src, amax_out, (uint32_t)items, ffn_hidden, per_row);
    swiglu_quant_kernel<<<grid_for(items), THREADS, 0, s>>>(src, amax_out, scale_out, q, (uint32_t)items, ffn_hidden, per_row);
    return (int)cudaGetLastError();
}

int fp8_quantize_bf16(const void* x_bf16, uint8_t* q, float* scale_out, const float* amax_in, size_t n, void* stream) {
    if (!x_bf16 || !q || !scale_out || !amax_in || (n % 16) != 0 || misaligned32(x_bf16) || misaligned(q)) return (int)cudaErrorInvalidValue;
    quant_bf16_kernel<<<grid_for(n / 32 + 1), THREADS, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint16_t*>(x_bf16), amax_in, scale_out, q,
                                                                                 n / 16);
    return (int)cudaGetLastError();
}

int fp8_residual_add(float* x, const void* y_bf16, size_t n, void* stream) {
    if (!x || !y_bf16 || (n % 8) != 0 || misaligned(x) || misaligned(y_bf16)) return (int)cudaErrorInvalidValue;
    if (n == 0) return 0;
    residual_add_kernel<<<grid_for(n / 8), THREADS, 0, (cudaStream_t)stream>>>(x, reinterpret_cast<const uint16_t*>(y_bf16), n / 8);
    return (int)cudaGetLastError();
}

}  // extern "C"
