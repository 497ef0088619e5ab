// fp8_gemm_mx_sm100.cu — block-scaled FP8 GEMM for NVIDIA B200 (sm_100a):
//     C[M,N] = alpha * sum over 32-element K blocks of  2^(ea[m,kb] + eb[n,kb]) * A[m, kb] . B[n, kb]
// with e4m3 elements and one ue8m0 scale per 32 elements along K for every row of A and of B (the OCP "MXFP8" format),
// multiplied by the tensor core itself: tcgen05.mma kind::mxf8f6f4.block_scale reads the scales from tensor memory.
// This is the step goml's roadmap names after its FP8 GEMM (docs/FP8_FA_ROADMAP.md:137-148: kind::mxf8f6f4
// .block_scale.scale_vec::1X, ue8m0 per 32 elements); the reference has no implementation of it.
//
// Data path of one work item: a 256 x 128 block of C as two 128-row halves that share the B operand, K swept in 128-byte
// slabs (four scale blocks):
//   TMA            the A slabs of both halves and the B slab (128 x 128 B each, 128-byte swizzle) and their 512-byte scale
//                  chunks (plain bulk copies) land in one ring stage; 4 stages
//   tcgen05.cp     the scale chunks go from shared memory to tensor memory (32 lanes x 128 bit, replicated over the four
//                  lane quarters: the layout the MMA reads — row r of a half finds its four scales at column r / 32)
//   tcgen05.mma    per half four M128 x N128 x K32 MMAs per slab, each selecting its scale byte (a_sf_id = b_sf_id =
//                  k-block): 8 MMAs = 512 tensor clocks per stage hand-shake, 48 KB of operands per 256 x 128 x 128 block
//   epilogue       8 warps; fp32 accumulators x alpha -> bf16 / fp16 -> global.  Tensor memory holds three 128-column
//                  accumulator slots used as a ring by consecutive halves, so the first half of the next item accumulates
//                  while the previous item drains, and the scale ring behind them
// The items of the last, partial wave over the SMs are single halves when that lets every SM finish in half an item's time.
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

constexpr int BM = 128, BN = 128, BK = 128;   // one half: 128 rows; an item has up to two halves
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, SF_BYTES = 512;
constexpr int OFF_B = 2 * A_BYTES, OFF_SF = 2 * A_BYTES + B_BYTES;   // stage: A half 0 | A half 1 | B | scales of A0, A1, B
constexpr int STAGE_BYTES = OFF_SF + 2048;                           // 51200: operand tiles stay 1024-byte aligned
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-9: epilogue
constexpr int TMEM_COLS = 512;        // accumulator slots [0, 384), scale ring [384, 384 + 16 * STAGES)
constexpr int ACC_SLOTS = 3;
constexpr int SF_COL = ACC_SLOTS * BN;
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
    int m_tiles, n_tiles, k_stages;   // 128-row tiles of A, 128-row tiles of B, 128-byte slabs of K
    int full_items;                   // items [0, full_items) are whole 256-row units
    int num_items;                    // the rest: single halves (split_tail) or whole units
    int split_tail;
};

// work item -> first 128-row tile of A, number of halves (0: nothing there), 128-row tile of B
struct Item { int rt, nh, tn; };
__device__ __forceinline__ Item decode_item(const MxParams& p, int idx) {
    Item it;
    if (idx < p.full_items || !p.split_tail) {
        it.rt = 2 * (idx / p.n_tiles);
        it.tn = idx % p.n_tiles;
        it.nh = min(2, p.m_tiles - it.rt);
    } else {
        const int j = idx - p.full_items;
        const int u = p.full_items + (j >> 1);
        it.rt = 2 * (u / p.n_tiles) + (j & 1);
        it.tn = u % p.n_tiles;
        it.nh = it.rt < p.m_tiles ? 1 : 0;
    }
    return it;
}

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
    const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES, bar_tfull = bars + 16 * STAGES, bar_tempty = bar_tfull + 8 * ACC_SLOTS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 16 * STAGES + 16 * ACC_SLOTS + 16);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < ACC_SLOTS; b++) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, NUM_EPI_WARPS); }
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
        // ------------------------------------------------------ TMA producer (whole warp; one elected lane issues)
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 1;  // "previous phase complete": the ring starts empty
            bool ok = true;
            for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
                const Item it = decode_item(p, idx);
                if (it.nh == 0) continue;
                const uint32_t tx = (uint32_t)it.nh * (A_BYTES + SF_BYTES) + B_BYTES + SF_BYTES;
                for (int ks = 0; ks < p.k_stages; ks++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    const uint32_t fb = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    if (leader) {
                        mbar_arrive_expect_tx(fb, tx);
                        for (int h = 0; h < it.nh; h++) {
                            tma_load_2d(sa + h * A_BYTES, &tmap_a, fb, ks * BK, (it.rt + h) * BM);   // rows past M: zero-filled
                            bulk_load(sa + OFF_SF + h * SF_BYTES, p.sfa + ((size_t)(it.rt + h) * p.k_stages + ks) * SF_BYTES, SF_BYTES, fb);
                        }
                        tma_load_2d(sa + OFF_B, &tmap_b, fb, ks * BK, it.tn * BN);
                        bulk_load(sa + OFF_SF + 2 * SF_BYTES, p.sfb + ((size_t)it.tn * p.k_stages + ks) * SF_BYTES, SF_BYTES, fb);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer (whole warp; one elected lane issues)
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            uint32_t cnt = 0;    // halves started so far: half c accumulates in slot c % 3, on that slot's use c / 3
            bool ok = true;
            for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
                const Item it = decode_item(p, idx);
                if (it.nh == 0) continue;
                for (int ks = 0; ks < p.k_stages && ok; ks++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    const uint32_t sf_tmem = tmem_base + SF_COL + 16 * stage;
                    // scale chunks: 32 rows of 16 bytes, no swizzle (8-row groups 128 bytes apart); the copies and the MMAs
                    // below run in issue order, so a stage's scales are in place before its MMAs and are not overwritten
                    // before the MMAs of the ring's previous lap have read them
                    for (int h = 0; h < it.nh; h++)
                        if (leader) tmem_cp_32x128b_warpx4(sf_tmem + 4 * h, make_smem_desc(sa + OFF_SF + h * SF_BYTES, 128, 128, LAYOUT_NONE));
                    if (leader) tmem_cp_32x128b_warpx4(sf_tmem + 8, make_smem_desc(sa + OFF_SF + 2 * SF_BYTES, 128, 128, LAYOUT_NONE));
                    const uint64_t bdesc = kmajor_desc_sw128(sa + OFF_B);
                    for (int h = 0; h < it.nh; h++) {
                        const uint32_t c = cnt + h, slot = c % ACC_SLOTS;
                        if (ks == 0) {   // the slot's previous contents must have been read out
                            if (!mbar_wait(bar_tempty + 8 * slot, ((c / ACC_SLOTS) & 1) ^ 1, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                            tc_fence_after();
                        }
                        const uint32_t d_tmem = tmem_base + slot * BN;
                        const uint64_t adesc = kmajor_desc_sw128(sa + h * A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 32; k++)   // +32 bytes along K inside the swizzle span = +2 in the address field
                            if (leader) mma_mx(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_mx(k), sf_tmem + 4 * h, sf_tmem + 8, (ks | k) != 0);
                    }
                    if (!ok) break;
                    if (leader) mma_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs retire
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok)
                    for (int h = 0; h < it.nh; h++) if (leader) mma_commit(bar_tfull + 8 * ((cnt + h) % ACC_SLOTS));  // accumulators complete
                cnt += it.nh;
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int chalf = (warp - 2) >> 2;         // which 64 columns of the half this warp converts
        const int row_in_tile = quad * 32 + lane;  // TMEM lane = row of the half
        const bool vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        uint32_t cnt = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
            const Item it = decode_item(p, idx);
            for (int h = 0; h < it.nh; h++, cnt++) {
                const uint32_t slot = cnt % ACC_SLOTS;
                if (!mbar_wait(bar_tfull + 8 * slot, (cnt / ACC_SLOTS) & 1, abort_flag, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
                tc_fence_after();
                const int row = (it.rt + h) * BM + row_in_tile;
                const uint32_t taddr = tmem_base + slot * BN + chalf * 64 + (uint32_t(quad * 32) << 16);
                uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + (size_t)row * p.N;
                if ((it.rt + h) * BM + quad * 32 < p.M) {       // else all 32 rows of this warp lie past M
#pragma unroll 1
                    for (int c = 0; c < 2; c++) {
                        const int col0 = it.tn * BN + chalf * 64 + c * 32;
                        if (col0 >= p.N) break;        // uniform across the warp
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
                                        if (p.out_bf16) { __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b); w[i] = *reinterpret_cast<uint32_t*>(&h2); }
                                        else { __half2 h2 = __floats2half2_rn(a, b); w[i] = *reinterpret_cast<uint32_t*>(&h2); }
                                    }
                                    *reinterpret_cast<uint4*>(crow + col0 + 8 * v) = make_uint4(w[0], w[1], w[2], w[3]);
                                }
                            } else {
                                for (int i = 0; i < 32 && col0 + i < p.N; i++) {
                                    const float a = __uint_as_float(acc[i]) * p.alpha;
                                    if (p.out_bf16) { __nv_bfloat16 h1 = __float2bfloat16_rn(a); crow[col0 + i] = *reinterpret_cast<uint16_t*>(&h1); }
                                    else { __half h1 = __float2half_rn(a); crow[col0 + i] = *reinterpret_cast<uint16_t*>(&h1); }
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * slot);   // this warp is done with the accumulator slot
            }
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
    const long long units = (long long)((p.m_tiles + 1) / 2) * p.n_tiles;
    if (units >= (1ll << 29)) return (int)cudaErrorInvalidValue;
    // whole waves of 256-row units over the SMs; the units of the last, partial wave go out as single halves when there
    // are few enough of them for every SM to take at most one
    const long long tail = units % st.num_sms;
    p.split_tail = (tail > 0 && 2 * tail <= st.num_sms) ? 1 : 0;
    p.full_items = p.split_tail ? (int)(units - tail) : (int)units;
    p.num_items = p.split_tail ? (int)(units + tail) : (int)units;
    CUtensorMap ta, tb;
    if (!make_tmap_u8_2d(&ta, A, (uint64_t)M, (uint64_t)K, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_tmap_u8_2d(&tb, B, (uint64_t)N, (uint64_t)K, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;
    const int grid = p.num_items < st.num_sms ? p.num_items : st.num_sms;
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
