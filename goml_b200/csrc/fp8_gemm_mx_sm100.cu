// fp8_gemm_mx_sm100.cu — block-scaled FP8 GEMM for NVIDIA B200 (sm_100a):
//     C[M,N] = alpha * sum over 32-element K blocks of  2^(ea[m,kb] + eb[n,kb]) * A[m, kb] . B[n, kb]
// with e4m3 elements and one ue8m0 scale per 32 elements along K for every row of A and of B (the OCP "MXFP8" format),
// multiplied by the tensor core itself: tcgen05.mma kind::mxf8f6f4.block_scale reads the scales from tensor memory.
// This is the step goml's roadmap names after its FP8 GEMM (docs/FP8_FA_ROADMAP.md:137-148: kind::mxf8f6f4
// .block_scale.scale_vec::1X, ue8m0 per 32 elements); the reference has no implementation of it.
//
// Data path of one 128 x 128 output tile, K swept in 128-byte slabs (four scale blocks):
//   TMA            A and B slabs (128 x 128 B each, 128-byte swizzle) and the two 512-byte scale chunks of the slab
//                  (plain bulk copies) land in one ring stage; 5 stages
//   tcgen05.cp     the scale chunks go from shared memory to tensor memory (32 lanes x 128 bit, replicated over the four
//                  lane quarters: the layout the MMA reads — row r of the tile finds its four scales at column r / 32)
//   tcgen05.mma    four M128 x N128 x K32 MMAs per slab, each selecting its scale byte (a_sf_id = b_sf_id = k-block)
//   epilogue       fp32 accumulators (double buffered in tensor memory) x alpha -> bf16 / fp16 -> global
// Scale arrays are stored in the chunk order the copy wants: for row tile rt and slab ks the 512 bytes at
// (rt * K/128 + ks) * 512 hold, at byte (l * 16 + c * 4 + kb), the scale of row rt*128 + 32 c + l and K block 4 ks + kb.
// Every mbarrier wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/fp8_gemm.h"
#include "sm100_ptx.cuh"
#include "tmap.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BN = 128, BK = 128;
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, SF_BYTES = 512;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;   // 33792: operand tiles stay 1024-byte aligned
constexpr int NUM_THREADS = 192;      // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int TMEM_COLS = 512;        // accumulators [0, 256), scale ring [256, 256 + 8 * STAGES)
constexpr int SF_COL = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

enum : uint32_t { ST_TIMEOUT_PRODUCER = 0x111, ST_TIMEOUT_MMA = 0x112, ST_TIMEOUT_EPILOGUE = 0x113 };

__device__ uint32_t g_mx_status = 0;

struct MxParams {
    int M, N, K;
    void* C;
    const uint8_t* sfa;
    const uint8_t* sfb;
    float alpha;
    int out_bf16;
    int m_tiles, n_tiles, k_stages;
};

// Instruction descriptor of the block-scaled kinds: [4,6) scale byte of B, [7,10) A format (0 = e4m3), [10,13) B format,
// [15] A major, [16] B major, [17,23) N >> 3, [23] scale format (1 = ue8m0), [24,29) M >> 4, [29,31) scale byte of A
__device__ __forceinline__ uint32_t idesc_mx(int k_block) {
    return ((uint32_t)k_block << 4) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) | ((uint32_t)(BM >> 4) << 24) | ((uint32_t)k_block << 29);
}
__device__ __forceinline__ void mma_mx(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, the same data in each of the four lane quarters
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
fp8_gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const MxParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + STAGES * STAGE_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES, bar_tfull = bars + 16 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 16 * STAGES + 32);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 4); }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 1;  // "previous phase complete": the ring starts empty
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int tm = t / p.n_tiles, tn = t - tm * p.n_tiles;
                for (int ks = 0; ks < p.k_stages; ks++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    const uint32_t fb = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(fb, STAGE_BYTES);
                    tma_load_2d(sa, &tmap_a, fb, ks * BK, tm * BM);              // rows past M: zero-filled
                    tma_load_2d(sa + A_BYTES, &tmap_b, fb, ks * BK, tn * BN);
                    bulk_load(sa + A_BYTES + B_BYTES, p.sfa + ((size_t)tm * p.k_stages + ks) * SF_BYTES, SF_BYTES, fb);
                    bulk_load(sa + A_BYTES + B_BYTES + SF_BYTES, p.sfb + ((size_t)tn * p.k_stages + ks) * SF_BYTES, SF_BYTES, fb);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t tphase[2] = {1, 1};  // both accumulator buffers start free
            int buf = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(bar_tempty + 8 * buf, tphase[buf], abort_flag, ST_TIMEOUT_MMA)) break;
                tphase[buf] ^= 1;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int ks = 0; ks < p.k_stages; ks++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    const uint32_t sf_tmem = tmem_base + SF_COL + 8 * stage;
                    // scale chunks: 32 rows of 16 bytes, no swizzle (8-row groups 128 bytes apart); the copies and the MMAs
                    // below run in issue order, so a stage's scales are in place before its MMAs and are not overwritten
                    // before the MMAs of the ring's previous lap have read them
                    tmem_cp_32x128b_warpx4(sf_tmem, make_smem_desc(sa + A_BYTES + B_BYTES, 128, 128, LAYOUT_NONE));
                    tmem_cp_32x128b_warpx4(sf_tmem + 4, make_smem_desc(sa + A_BYTES + B_BYTES + SF_BYTES, 128, 128, LAYOUT_NONE));
                    const uint64_t adesc = kmajor_desc_sw128(sa);
                    const uint64_t bdesc = kmajor_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 32; k++)   // +32 bytes along K inside the swizzle span = +2 in the address field
                        mma_mx(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_mx(k), sf_tmem, sf_tmem + 4, (ks | k) != 0);
                    mma_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) mma_commit(bar_tfull + 8 * buf);  // accumulator complete
                buf ^= 1;
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;  // TMEM lane = row of the tile
        const bool vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        uint32_t tphase[2] = {0, 0};
        int buf = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const int tm = t / p.n_tiles, tn = t - tm * p.n_tiles;
            if (!mbar_wait(bar_tfull + 8 * buf, tphase[buf], abort_flag, ST_TIMEOUT_EPILOGUE)) break;
            tphase[buf] ^= 1;
            tc_fence_after();
            const int row = tm * BM + row_in_tile;
            const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quad * 32) << 16);
            uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + (size_t)row * p.N;
            if (tm * BM + quad * 32 < p.M) {       // else all 32 rows of this warp lie past M
#pragma unroll 1
                for (int c = 0; c < BN / 32; c++) {
                    const int col0 = tn * BN + c * 32;
                    if (col0 >= p.N) break;        // uniform across the CTA
                    uint32_t acc[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, acc);
                    tmem_ld_wait();
                    if (row < p.M) {
                        if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                            for (int v = 0; v < 4; v++) {
                                uint32_t w[4];
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const float a = __uint_as_float(acc[8 * v + 2 * i]) * p.alpha, b = __uint_as_float(acc[8 * v + 2 * i + 1]) * p.alpha;
                                    if (p.out_bf16) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); w[i] = *reinterpret_cast<uint32_t*>(&h); }
                                    else { __half2 h = __floats2half2_rn(a, b); w[i] = *reinterpret_cast<uint32_t*>(&h); }
                                }
                                *reinterpret_cast<uint4*>(crow + col0 + 8 * v) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
                            for (int i = 0; i < 32 && col0 + i < p.N; i++) {
                                const float a = __uint_as_float(acc[i]) * p.alpha;
                                if (p.out_bf16) { __nv_bfloat16 h = __float2bfloat16_rn(a); crow[col0 + i] = *reinterpret_cast<uint16_t*>(&h); }
                                else { __half h = __float2half_rn(a); crow[col0 + i] = *reinterpret_cast<uint16_t*>(&h); }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);   // this warp is done with the accumulator buffer
            buf ^= 1;
        }
    }

    // ------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    const uint32_t code = *abort_flag;
    if (code != 0) {
        if (threadIdx.x == 0) atomicCAS(&g_mx_status, 0u, code);
        for (int i = 0; i < 200; i++) __nanosleep(1000);   // let copies already in flight land
        __syncthreads();
    }
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

struct DeviceState {
    std::once_flag once;
    cudaError_t init_error = cudaSuccess;
    int num_sms = 0;
};
DeviceState g_dev[64];

void init_device(DeviceState* st, int dev) {
    int major = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess && major != 10) e = cudaErrorNoKernelImageForDevice;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&st->num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fp8_gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    st->init_error = e;
}

}  // namespace

extern "C" {

size_t fp8_mx_scale_bytes(int rows, int K) {
    if (rows <= 0 || K <= 0) return 0;
    return (size_t)((rows + 127) / 128) * (size_t)((K + 127) / 128) * 512;
}

int fp8_gemm_mx(int M, int N, int K, const void* A, const void* scale_a, const void* B, const void* scale_b, void* C, float alpha,
                int out_dtype, void* stream) {
    if (M < 0 || N < 0 || K < 0) return (int)cudaErrorInvalidValue;
    if (M == 0 || N == 0) return 0;
    if (!A || !B || !C || !scale_a || !scale_b) return (int)cudaErrorInvalidValue;
    if (K == 0 || (K % 128) != 0) return (int)cudaErrorInvalidValue;     // whole 128-element slabs (four scale blocks)
    if (out_dtype != FP8_GEMM_OUT_FP16 && out_dtype != FP8_GEMM_OUT_BF16) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(scale_a) & 15) ||
        (reinterpret_cast<uintptr_t>(scale_b) & 15) || (reinterpret_cast<uintptr_t>(C) & 1))
        return (int)cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    DeviceState& st = g_dev[dev];
    std::call_once(st.once, init_device, &st, dev);
    if (st.init_error != cudaSuccess) return (int)st.init_error;

    MxParams p;
    p.M = M; p.N = N; p.K = K; p.C = C;
    p.sfa = static_cast<const uint8_t*>(scale_a); p.sfb = static_cast<const uint8_t*>(scale_b);
    p.alpha = alpha; p.out_bf16 = out_dtype == FP8_GEMM_OUT_BF16;
    p.m_tiles = (M + BM - 1) / BM; p.n_tiles = (N + BN - 1) / BN; p.k_stages = K / BK;
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles >= (1ll << 30)) return (int)cudaErrorInvalidValue;
    CUtensorMap ta, tb;
    if (!make_tmap_u8_2d(&ta, A, (uint64_t)M, (uint64_t)K, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_tmap_u8_2d(&tb, B, (uint64_t)N, (uint64_t)K, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;
    const int grid = (int)(tiles < st.num_sms ? tiles : st.num_sms);
    fp8_gemm_mx_kernel<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, p);
    return (int)cudaGetLastError();
}

int fp8_gemm_mx_device_status(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return -(int)e;
    uint32_t code = 0, zero = 0;
    e = cudaMemcpyFromSymbol(&code, g_mx_status, sizeof(code));
    if (e != cudaSuccess) return -(int)e;
    if (code != 0) cudaMemcpyToSymbol(g_mx_status, &zero, sizeof(zero));
    return (int)code;
}

}  // extern "C"
