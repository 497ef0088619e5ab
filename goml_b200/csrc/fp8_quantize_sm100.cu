// fp8_quantize_sm100.cu — libfp8quant.so: per-tensor FP32 -> e4m3 quantiser
// (amax reduction + scale + round-to-nearest-even, saturating conversion).
// HBM-bound: the amax pass reads 4 B/element, the conversion pass reads 4 B and
// writes 1 B per element (the second read is served from L2 when the tensor
// fits).  128-bit loads, one 128-bit store per 16 elements, grid sized to a
// multiple of the SM count.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fp8_quantize.h"

namespace {

constexpr int THREADS = 256;

__global__ void __launch_bounds__(THREADS) amax_kernel(const float* __restrict__ x, size_t n, float* amax) {
    const size_t n4 = n / 4;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float m = 0.f;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(x4 + i);
        m = fmaxf(fmaxf(m, fabsf(v.x)), fmaxf(fabsf(v.y), fmaxf(fabsf(v.z), fabsf(v.w))));  // NaN never wins
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) m = fmaxf(m, fabsf(x[n4 * 4 + threadIdx.x]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float wm[THREADS / 32];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < THREADS / 32 ? wm[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        // non-negative floats order like their bit patterns
        if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));
    }
}

__device__ __forceinline__ uint32_t quant4(float4 v, float inv) {
    // x * inv (one rounding, no FMA contraction possible), clamp, RN-even satfinite
    const float a = fminf(fmaxf(__fmul_rn(v.x, inv), -448.f), 448.f);
    const float b = fminf(fmaxf(__fmul_rn(v.y, inv), -448.f), 448.f);
    const float c = fminf(fmaxf(__fmul_rn(v.z, inv), -448.f), 448.f);
    const float d = fminf(fmaxf(__fmul_rn(v.w, inv), -448.f), 448.f);
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__global__ void __launch_bounds__(THREADS) quant_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, size_t n,
                                                        const float* __restrict__ amax_ptr, float* scale_out,
                                                        float divisor) {
    const float amax = *amax_ptr;
    const float scale = (amax > 1e-12f) ? __fdiv_rn(amax, divisor) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const size_t n16 = n / 16;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    uint4* q16 = reinterpret_cast<uint4*>(q);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const float4 a = __ldg(x4 + 4 * i), b = __ldg(x4 + 4 * i + 1), c = __ldg(x4 + 4 * i + 2), d = __ldg(x4 + 4 * i + 3);
        q16[i] = make_uint4(quant4(a, inv), quant4(b, inv), quant4(c, inv), quant4(d, inv));
    }
    if (blockIdx.x == 0) {
        for (size_t i = n16 * 16 + threadIdx.x; i < n; i += blockDim.x) {
            const float v = fminf(fmaxf(__fmul_rn(x[i], inv), -448.f), 448.f);
            q[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
        }
    }
}

__global__ void __launch_bounds__(THREADS) dequant_kernel(const uint8_t* __restrict__ q, __half* __restrict__ out,
                                                          const float* __restrict__ scale_in, int n) {
    const float s = *scale_in;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(q[i], __NV_E4M3);
        out[i] = __float2half_rn(__half2float(__half(hr)) * s);
    }
}

// ---- FP16 sources: the reference's own entry point (libs1/fp8_quantize_v2.cu:176-204) has no stream, no amax
// argument and allocates its reduction buffer itself; here the amax word is a per-GPU device variable, so the
// entry allocates nothing.  Calls run on the legacy default stream like the reference's and therefore serialise.
__device__ float g_amax_fp16;

__global__ void clear_amax_fp16_kernel() { g_amax_fp16 = 0.f; }

__global__ void __launch_bounds__(THREADS) amax_fp16_kernel(const __half* __restrict__ x, int n) {
    // 8 halves (16 bytes) per step when the pointer allows it, else element by element
    float m = 0.f;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const size_t n8 = (size_t)n / 8;
        const uint4* x8 = reinterpret_cast<const uint4*>(x);
        for (size_t i = tid; i < n8; i += stride) {
            const uint4 v = __ldg(x8 + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
        for (size_t i = n8 * 8 + tid; i < (size_t)n; i += stride) m = fmaxf(m, fabsf(__half2float(x[i])));
    } else {
        for (size_t i = tid; i < (size_t)n; i += stride) m = fmaxf(m, fabsf(__half2float(x[i])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float wm[THREADS / 32];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < THREADS / 32 ? wm[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(&g_amax_fp16), __float_as_uint(m));
    }
}

__global__ void __launch_bounds__(THREADS) quant_fp16_kernel(const __half* __restrict__ x, uint8_t* __restrict__ q, int n,
                                                             float* scale_out) {
    // operation order of libs1/fp8_quantize_v2.cu:89-121: scale = amax / 448, inv = 1 / scale, v = float(x) * inv,
    // clamp to +-448, round to nearest even
    const float amax = g_amax_fp16;
    const float scale = (amax > 1e-12f) ? __fdiv_rn(amax, 448.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
    const size_t n8 = vec ? (size_t)n / 8 : 0;
    const uint4* x8 = reinterpret_cast<const uint4*>(x);
    uint2* q8 = reinterpret_cast<uint2*>(q);
    for (size_t i = tid; i < n8; i += stride) {
        const uint4 v = __ldg(x8 + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t c[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            const float a = fminf(fmaxf(__fmul_rn(f.x, inv), -448.f), 448.f);
            const float b = fminf(fmaxf(__fmul_rn(f.y, inv), -448.f), 448.f);
            c[k] = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        }
        q8[i] = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
    }
    for (size_t i = n8 * 8 + tid; i < (size_t)n; i += stride) {
        const float v = fminf(fmaxf(__fmul_rn(__half2float(x[i]), inv), -448.f), 448.f);
        q[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    }
}

// ---- block-scaled ("MXFP8") quantiser: one ue8m0 scale per 32 consecutive elements of a row (OCP microscaling:
// scale = 2^(floor(log2(amax)) - 8), 8 = the largest e4m3 exponent; elements = e4m3_rn_satfinite(x / scale)).
// One thread per block of 32: 128 bytes read, 32 codes and one scale byte written; the scale byte goes to the tiled
// position the block-scaled GEMM copies from (fp8_gemm.h: fp8_gemm_mx).
__global__ void __launch_bounds__(THREADS) quant_mx_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                           int rows, int K) {
    const int kblocks = K / 32;
    const size_t total = (size_t)rows * kblocks;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int row = (int)(i / kblocks), kb = (int)(i - (size_t)row * kblocks);
        const float4* src = reinterpret_cast<const float4*>(x + (size_t)row * K + kb * 32);
        float4 v[8];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            v[j] = __ldg(src + j);
            amax = fmaxf(fmaxf(amax, fabsf(v[j].x)), fmaxf(fabsf(v[j].y), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));  // NaN never wins
        }
        int se = 0;                                   // an all-zero block keeps scale 1
        if (amax > 0.f && amax <= 3.4028234e38f) se = ilogbf(amax) - 8;
        else if (amax > 3.4028234e38f) se = 127;      // infinity in the block
        se = max(-127, min(127, se));
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // x * 2^-se is exact (a change of exponent) unless the result is subnormal in fp32
            const float a = fminf(fmaxf(scalbnf(v[j].x, -se), -448.f), 448.f), b = fminf(fmaxf(scalbnf(v[j].y, -se), -448.f), 448.f);
            const float c = fminf(fmaxf(scalbnf(v[j].z, -se), -448.f), 448.f), d = fminf(fmaxf(scalbnf(v[j].w, -se), -448.f), 448.f);
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
            w[j] = lo | (hi << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(q + (size_t)row * K + kb * 32);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        const size_t chunk = (size_t)(row >> 7) * (K / 128) + (kb >> 2);
        sf[chunk * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3)] = (uint8_t)(se + 127);
    }
}

int grid_for(size_t work_items) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t blocks = (work_items + THREADS - 1) / THREADS;
    const size_t cap = (size_t)sms * 8;  // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

extern "C" {

int fp8_quantize_f32(const float* x, uint8_t* q, float* scale_out, float* amax_out, size_t n, int convention,
                     void* stream) {
    if (!x || !q || !scale_out || !amax_out) return (int)cudaErrorInvalidValue;
    if (convention != FP8_QUANT_AMAX_OVER_448 && convention != FP8_QUANT_UNIT) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    if (n > 0) amax_kernel<<<grid_for(n / 4 + 1), THREADS, 0, s>>>(x, n, amax_out);
    quant_kernel<<<grid_for(n / 16 + 1), THREADS, 0, s>>>(x, q, n, amax_out, scale_out,
                                                           convention == FP8_QUANT_UNIT ? 1.0f : 448.0f);
    return (int)cudaGetLastError();
}

int fp8_dequantize_to_fp16(const void* input_fp8, void* output_fp16, const float* scale_in, int n) {
    if (!input_fp8 || !output_fp16 || !scale_in || n < 0) return (int)cudaErrorInvalidValue;
    if (n == 0) return 0;
    dequant_kernel<<<grid_for((size_t)n), THREADS>>>((const uint8_t*)input_fp8, (__half*)output_fp16, scale_in, n);
    return (int)cudaGetLastError();
}

int fp8_quantize_fp16(const void* input_fp16, void* output_fp8, float* scale_out, int n) {
    if (!input_fp16 || !output_fp8 || !scale_out || n < 0) return (int)cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(input_fp16) & 1) return (int)cudaErrorInvalidValue;
    clear_amax_fp16_kernel<<<1, 1>>>();
    if (n > 0) amax_fp16_kernel<<<grid_for((size_t)n / 8 + 1), THREADS>>>((const __half*)input_fp16, n);
    quant_fp16_kernel<<<grid_for((size_t)n / 8 + 1), THREADS>>>((const __half*)input_fp16, (uint8_t*)output_fp8, n, scale_out);
    return (int)cudaGetLastError();
}

int cuda_device_sync2(void) { return (int)cudaDeviceSynchronize(); }

int fp8_quantize_mx_f32(const float* x, uint8_t* q, uint8_t* scales, int rows, int K, void* stream) {
    if (!x || !q || !scales || rows < 0 || K <= 0 || (K % 128) != 0) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15)) return (int)cudaErrorInvalidValue;
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    // entries of the padding rows of the last 128-row tile: scale 1 (never the NaN byte)
    const size_t sf_bytes = (size_t)((rows + 127) / 128) * (size_t)(K / 128) * 512;
    cudaError_t e = cudaMemsetAsync(scales, 0x7f, sf_bytes, s);
    if (e != cudaSuccess) return (int)e;
    quant_mx_kernel<<<grid_for((size_t)rows * (K / 32)), THREADS, 0, s>>>(x, q, scales, rows, K);
    return (int)cudaGetLastError();
}

}  // extern "C"
