// fp8_gemm_sm100.cu — libfp8gemm.so for NVIDIA B200 (sm_100a).
//
//   C[M,N] = alpha * A[M,K] . B[N,K]^T     A, B: e4m3 codes, K contiguous; C: fp16 or bf16
//
// Drop-in for goml's libs/fp8_gemm.cu:308-355 (same three exported symbols,
// same argument meaning and return convention), rebuilt around the Blackwell
// data path instead of mma.sync:
//
//   TMA (128-byte swizzle) -> 4-stage shared-memory ring under mbarriers (6 stages / 4 double stages for the narrower tiles)
//     -> one thread issues tcgen05.mma kind::f8f6f4 (M128 x N256 x K32), FP32
//        accumulators in tensor memory, double buffered (2 x 256 columns)
//     -> 4 epilogue warps read TMEM (tcgen05.ld), scale, convert and store with
//        128-bit stores while the next tile's main loop already runs.
//
// One persistent CTA per SM walks output tiles in an order that keeps a band of
// A rows and a few B panels resident in L2.  Every CTA loads its own tiles; no thread-block clusters.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "../../include/fp8_gemm.h"
#include "sm100_ptx.cuh"
#include "tmap.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;          // rows of C per tile (= TMEM lanes)
constexpr int BK = 128;          // K bytes per pipeline stage (one 128-byte swizzle span)
constexpr int A_BYTES = BM * BK;
constexpr int NUM_THREADS = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int GROUP_M = 16;       // tile-order band height (in tiles)
// epilogue staging for the fp32 accumulate mode: per epilogue warp two 32-row x 128-byte boxes (128-byte swizzle)
constexpr int STAGING_BOX = 32 * 128;
constexpr int STAGING_BYTES = 4 * 2 * STAGING_BOX;

// Tile width BN (columns of C per tile = TMEM columns per accumulator buffer).  256 is the
// tensor-efficient shape (the MMA reads (128+BN)*32 operand bytes per BN/2 clocks, within the
// 128 B/clk shared-memory read rate only for BN >= 128); 128 and 64 exist so that small and
// skinny problems (few 128x256 tiles) still spread over all SMs — those are HBM/latency-bound,
// and a narrower tile leaves room for a deeper TMA ring.
// MT = 2: a CTA works on a pair of vertically adjacent tiles (256 rows) that share every B tile it loads.
template <int BN, int MT = 1>
struct Tile {
    static constexpr int B_BYTES = BN * BK;
    // The narrow tile serves HBM-bound problems whose MMAs take only 192 clk per k-block: there the producer's and the
    // issuer's per-stage work (a wait, an expect / a commit) is the bound, so a stage holds two k-blocks.
    static constexpr int KSUB = (BN == 64) ? 2 : 1;
    static constexpr int SUB_BYTES = MT * A_BYTES + B_BYTES;
    static constexpr int STAGE_BYTES = KSUB * SUB_BYTES;
    static constexpr int STAGES = (MT == 2) ? 3 : (BN == 256) ? 4 : (BN == 128) ? 6 : 4;
    static constexpr int TMEM_COLS = 2 * BN;  // two accumulator buffers (a power of two >= 32)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

enum : uint32_t {
    ST_OK = 0,
    ST_TIMEOUT_PRODUCER = 0x101,
    ST_TIMEOUT_MMA = 0x102,
    ST_TIMEOUT_EPILOGUE = 0x103,
    ST_TIMEOUT_SELFTEST = 0x1F0,   // fp8_gemm_selftest_wait_expiry
};

__device__ uint32_t g_gemm_status = 0;  // first non-zero code any CTA reported (per device)

struct GemmParams {
    int M, N, K;
    void* C;
    float alpha;
    const float* scale_a;
    const float* scale_b;
    int out_bf16;
    float* X;  // when set: X[M,N] (fp32) += alpha * A.B^T instead of storing C (the residual-stream update of a decoder block)
    // SwiGLU mode: B holds 32 gate rows then the 32 matching up rows per 64 rows, so every tile width holds whole
    // pairs; the epilogue writes H[M, F] = silu(alpha*gate) * (alpha*up) as bf16 and reduces max|H| into *amax
    void* H;
    int F;
    float* amax;
    // e4m3-output mode: D8[M,N] = e4m3(scale_d * v), v = alpha * A.B^T rounded to fp32, and max|v| reduced into *amax
    uint8_t* D8;
    const float* scale_d;
    int h_tma;  // SwiGLU output H likewise (F % 8 == 0); only tiles of 128 or 256 columns use it
    int d_tma;  // e4m3 output D likewise (N % 16 == 0); only tiles of 128 or 256 columns use it
    int c_tma;  // C (16-bit) can be described by a tensor map (16-byte aligned, N % 8 == 0): tiles leave through staging + TMA store
    int x_tma;  // X can be described by a tensor map (16-byte aligned, N % 4 == 0): add through TMA reduce, else read-modify-write
    int m_tiles, n_tiles, k_blocks;
    int split_from;  // tiles [split_from, m_tiles*n_tiles) of the last, less than half full wave run as two half-width units each
    int num_units;   // split_from + 2 * (number of split tiles); with ksplit > 1: tiles * ksplit
    // split-K (accumulate mode through TMA reduce only, where partial sums may simply be added into X): unit u is
    // slice u % ksplit of tile u / ksplit and covers pipeline stages [slice * ks_per, min((slice + 1) * ks_per, all))
    int ksplit, ks_per;
    // rows of A one TMA box brings in: 128, or for a single row of tiles with M <= 64 the next of 16 / 32 / 64, so a
    // skinny problem does not fill shared memory with 128-row tiles of mostly zero padding; the tile rows past it
    // keep whatever shared memory held (their accumulator rows are never stored or counted)
    int a_rows;
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& tm, int& tn) {
    const int per_group = GROUP_M * n_tiles;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(m_tiles - first_m, GROUP_M);
    const int r = t - g * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

// Work unit u -> tile coordinates, first column and width.  Units below split_from are whole tiles; above it,
// two consecutive units are the left and right halves of one tile (only instantiated for BN = 256).
template <int BN>
__device__ __forceinline__ void unit_coords(int u, const GemmParams& p, int& tm, int& n0, int& bn) {
    int t = u, half = -1;
    if (BN == 256 && u >= p.split_from) {
        t = p.split_from + ((u - p.split_from) >> 1);
        half = (u - p.split_from) & 1;
    }
    int tn;
    tile_coords(t, p.m_tiles, p.n_tiles, tm, tn);
    n0 = tn * BN;
    bn = BN;
    if (half >= 0) {
        bn = BN / 2;
        n0 += half * (BN / 2);
    }
}

__device__ __forceinline__ uint32_t pack_out(float a, float b, int bf16) {
    if (bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// four fp32 -> four e4m3 codes (round to nearest even, saturate to +-448, NaN -> 0x7f), a in the lowest byte
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

template <int BN, int MT = 1>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fp8_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_b_half, const __grid_constant__ CUtensorMap tmap_x,
                        const GemmParams p) {
    constexpr int STAGES = Tile<BN, MT>::STAGES;
    constexpr int STAGE_BYTES = Tile<BN, MT>::STAGE_BYTES;
    constexpr int TMEM_COLS = Tile<BN, MT>::TMEM_COLS;
    constexpr int KSUB = Tile<BN, MT>::KSUB;
    constexpr int SUB_BYTES = Tile<BN, MT>::SUB_BYTES;
    const int k_stages = (p.k_blocks + KSUB - 1) / KSUB;
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment (swizzle atom = 8 rows x 128 B)
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t staging = smem_base + STAGES * STAGE_BYTES;
    const uint32_t bars = staging + STAGING_BYTES;
    // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    const uint32_t bar_full = bars;
    const uint32_t bar_empty = bars + 8 * STAGES;
    const uint32_t bar_tfull = bars + 16 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + STAGES * STAGE_BYTES + STAGING_BYTES + 16 * STAGES + 32);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_units = p.num_units;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        // The whole warp runs the loop and one elected lane issues: coordinates and addresses stay warp-uniform.
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 1;  // "previous phase complete": the ring starts empty
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                int tm, n0, bn;
                const int t = u / p.ksplit, ks0 = (u - t * p.ksplit) * p.ks_per, ks1 = min(ks0 + p.ks_per, k_stages);
                unit_coords<BN>(t, p, tm, n0, bn);
                const CUtensorMap* tb = (bn == BN) ? &tmap_b : &tmap_b_half;
                for (int ks = ks0; ks < ks1; ks++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    const uint32_t fb = bar_full + 8 * stage;
                    if (leader) {
                        mbar_arrive_expect_tx(fb, KSUB * (MT * p.a_rows * BK + bn * BK));
#pragma unroll
                        for (int sub = 0; sub < KSUB; sub++) {
                            // a k-block past the end of K (odd count) is a fully out-of-range box: zero-filled, bytes still counted
                            const int kb = ks * KSUB + sub;
                            const uint32_t sa = smem_base + stage * STAGE_BYTES + sub * SUB_BYTES;
                            tma_load_2d(sa, &tmap_a, fb, kb * BK, MT * tm * BM);
                            if (MT == 2) tma_load_2d(sa + A_BYTES, &tmap_a, fb, kb * BK, (2 * tm + 1) * BM);   // past M: zero-filled
                            tma_load_2d(sa + MT * A_BYTES, tb, fb, kb * BK, n0);
                        }
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        // Whole warp, one elected lane issues (descriptors stay in uniform registers).
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            uint32_t tphase[2] = {1, 1};  // both accumulator buffers start free
            int buf = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const int t = u / p.ksplit, ks0 = (u - t * p.ksplit) * p.ks_per, ks1 = min(ks0 + p.ks_per, k_stages);
                const bool whole = !(BN == 256 && t >= p.split_from);
                const uint32_t idesc = whole ? make_idesc_e4m3_f32(BM, BN, 0, 0) : make_idesc_e4m3_f32(BM, BN / 2, 0, 0);
                if (MT == 2) buf = 0;   // a tile pair takes both accumulator buffers: upper half in 0, lower half in 1
                if (!mbar_wait(bar_tempty + 8 * buf, tphase[buf], abort_flag, ST_TIMEOUT_MMA)) break;
                tphase[buf] ^= 1;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int ks = ks0; ks < ks1; ks++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int sub = 0; sub < KSUB; sub++) {
                        const uint32_t sa = smem_base + stage * STAGE_BYTES + sub * SUB_BYTES;
                        const uint64_t adesc = kmajor_desc_sw128(sa);
                        const uint64_t bdesc = kmajor_desc_sw128(sa + MT * A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 32; k++) {
                            // +32 bytes along K inside the swizzle span = +2 in the address field
                            if (leader) mma_f8f6f4_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, ((ks - ks0) | sub | k) != 0);
                        }
                        if (MT == 2) {
                            // lower half of the pair: the other accumulator buffer, the same B operand.  Its buffer is
                            // waited for only here, so the epilogue of the previous pair's lower half overlaps the
                            // first MMAs of this pair's upper half.
                            if (ks == ks0 && sub == 0) {
                                if (!mbar_wait(bar_tempty + 8, tphase[1], abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                                tphase[1] ^= 1;
                                tc_fence_after();
                            }
                            const uint64_t adesc2 = kmajor_desc_sw128(sa + A_BYTES);
#pragma unroll
                            for (int k = 0; k < BK / 32; k++)
                                if (leader) mma_f8f6f4_ss(tmem_base + BN, adesc2 + 2 * k, bdesc + 2 * k, idesc, ((ks - ks0) | sub | k) != 0);
                        }
                    }
                    if (!ok) break;
                    if (leader) mma_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs retire
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok && leader) mma_commit(bar_tfull + 8 * buf);  // accumulator complete
                if (ok && leader && MT == 2) mma_commit(bar_tfull + 8);
                buf ^= 1;
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;  // TMEM lane = row of the tile
        float alpha = p.alpha;
        if (p.scale_a) alpha *= __ldg(p.scale_a);
        if (p.scale_b) alpha *= __ldg(p.scale_b);
        const bool vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        const bool xvec_ok = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.X) & 15) == 0);
        const bool dvec_ok = (p.N % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.D8) & 15) == 0);
        const float scale_d = (p.D8 && p.scale_d) ? __ldg(p.scale_d) : 1.0f;
        uint32_t tphase[2] = {0, 0};
        int buf = 0;
        int sbuf = 0;  // staging box in use (accumulate mode)
        for (int u = blockIdx.x; u < num_units; u += gridDim.x)
        for (int hsel = 0; hsel < MT; hsel++) {   // a tile pair is two tiles to the epilogue: buffer 0, then buffer 1
            int tm, n0, bn;
            unit_coords<BN>(u / p.ksplit, p, tm, n0, bn);
            tm = MT * tm + hsel;
            if (!mbar_wait(bar_tfull + 8 * buf, tphase[buf], abort_flag, ST_TIMEOUT_EPILOGUE)) goto epilogue_done;
            tphase[buf] ^= 1;
            tc_fence_after();
            const int row = tm * BM + row_in_tile;
            const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quad * 32) << 16);
            uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + (size_t)row * p.N;
            float tmax = 0.f;  // running max of this thread's row (SwiGLU and e4m3-output modes)
            if (tm * BM + quad * 32 >= p.M) {
                // all 32 rows of this warp lie past M (a skinny problem uses 16 of a tile's 128 rows): nothing to
                // read, convert or store; the accumulator buffer is handed back below as usual
            } else if (p.H) {
                // accumulator columns [64c, 64c+32) are gate and [64c+32, 64c+64) up of activation columns n0/2 + [32c, 32c+32)
                uint16_t* hrow = reinterpret_cast<uint16_t*>(p.H) + (size_t)row * p.F;
                const bool hvec_ok = (p.F % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.H) & 15) == 0);
#pragma unroll 1
                for (int c = 0; c < bn / 64; c++) {
                    const int col0 = (n0 >> 1) + c * 32;   // activation column of this chunk
                    if (col0 >= p.F) break;                 // uniform across the CTA
                    uint32_t g[32], uacc[32];
                    tmem_ld_32x32b_x32(taddr + c * 64, g);
                    tmem_ld_32x32b_x32(taddr + c * 64 + 32, uacc);
                    tmem_ld_wait();
                    uint32_t w[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        float h[2];
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const float gv = __uint_as_float(g[2 * j + e]) * alpha;
                            const float uv = __uint_as_float(uacc[2 * j + e]) * alpha;
                            float r;
                            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + __expf(-gv)));
                            h[e] = gv * r * uv;
                        }
                        const __nv_bfloat162 hb = __floats2bfloat162_rn(h[0], h[1]);
                        w[j] = *reinterpret_cast<const uint32_t*>(&hb);
                        // max of the rounded values = what the quantiser that follows will see
                        tmax = fmaxf(tmax, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xffff0000u))));
                    }
                    if (BN >= 128 && p.h_tma) {
                        // two 32-column chunks fill one 32 x 64 box of this warp's rows (every tile and half-tile is a
                        // whole number of boxes; past column F the tensor map clips), one TMA store per box
                        const uint32_t box = staging + (quad * 2 + sbuf) * STAGING_BOX;
                        if ((c & 1) == 0) {
                            if (lane == 0) tma_store_wait_read<1>();  // the store that used this buffer two boxes ago has read it
                            __syncwarp();
                        }
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            const uint32_t dst = box + lane * 128 + ((((c & 1) * 4 + v) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[4 * v]), "r"(w[4 * v + 1]), "r"(w[4 * v + 2]),
                                         "r"(w[4 * v + 3])
                                         : "memory");
                        }
                        if ((c & 1) || col0 + 32 >= p.F) {   // box complete, or no further chunk of this matrix
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                tma_store_2d(&tmap_x, box, col0 - (c & 1) * 32, tm * BM + quad * 32);
                                tma_store_commit();
                            }
                            sbuf ^= 1;
                        }
                    } else if (row < p.M) {
                        if (hvec_ok && col0 + 32 <= p.F) {
                            uint4* dst = reinterpret_cast<uint4*>(hrow + col0);
#pragma unroll
                            for (int v = 0; v < 4; v++) dst[v] = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (col0 + j < p.F) hrow[col0 + j] = (uint16_t)((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu));
                        }
                    }
                }
            } else if (BN >= 128 && p.d_tma) {
                // e4m3 D through the memory system: four 32-column chunks of this warp's 32 rows fill one 32 x 128 box
#pragma unroll 1
                for (int c4 = 0; c4 < bn / 128; c4++) {
                    const int col0 = n0 + c4 * 128;
                    if (col0 >= p.N) break;  // uniform across the CTA
                    const uint32_t box = staging + (quad * 2 + sbuf) * STAGING_BOX;
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        uint32_t acc[32];
                        tmem_ld_32x32b_x32(taddr + c4 * 128 + q4 * 32, acc);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            v[j] = __uint_as_float(acc[j]) * alpha;
                            tmax = fmaxf(tmax, fabsf(v[j]));   // columns >= N and rows >= M hold zeros
                            v[j] *= scale_d;
                        }
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const uint32_t dst = box + lane * 128 + (((q4 * 2 + h) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                         "r"(pack_e4m3x4(v[16 * h + 0], v[16 * h + 1], v[16 * h + 2], v[16 * h + 3])),
                                         "r"(pack_e4m3x4(v[16 * h + 4], v[16 * h + 5], v[16 * h + 6], v[16 * h + 7])),
                                         "r"(pack_e4m3x4(v[16 * h + 8], v[16 * h + 9], v[16 * h + 10], v[16 * h + 11])),
                                         "r"(pack_e4m3x4(v[16 * h + 12], v[16 * h + 13], v[16 * h + 14], v[16 * h + 15]))
                                         : "memory");
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_x, box, col0, tm * BM + quad * 32);
                        tma_store_commit();
                    }
                    sbuf ^= 1;
                }
            } else if (p.c_tma) {
                // 16-bit C through the memory system: two 32-column chunks of this warp's 32 rows fill one 32 x 64 box
                // (128-byte rows, swizzled like the fp32 boxes of the accumulate mode), one TMA store per box,
                // double-buffered; rows >= M and columns >= N are clipped by the tensor map
#pragma unroll 1
                for (int c2 = 0; c2 < bn / 64; c2++) {
                    const int col0 = n0 + c2 * 64;
                    if (col0 >= p.N) break;  // uniform across the CTA
                    const uint32_t box = staging + (quad * 2 + sbuf) * STAGING_BOX;
                    if (lane == 0) tma_store_wait_read<1>();  // the store that used this buffer two boxes ago has read it
                    __syncwarp();
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        uint32_t acc[32];
                        tmem_ld_32x32b_x32(taddr + c2 * 64 + hf * 32, acc);
                        tmem_ld_wait();
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            const uint32_t dst = box + lane * 128 + (((hf * 4 + v) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                         "r"(pack_out(__uint_as_float(acc[8 * v + 0]) * alpha, __uint_as_float(acc[8 * v + 1]) * alpha, p.out_bf16)),
                                         "r"(pack_out(__uint_as_float(acc[8 * v + 2]) * alpha, __uint_as_float(acc[8 * v + 3]) * alpha, p.out_bf16)),
                                         "r"(pack_out(__uint_as_float(acc[8 * v + 4]) * alpha, __uint_as_float(acc[8 * v + 5]) * alpha, p.out_bf16)),
                                         "r"(pack_out(__uint_as_float(acc[8 * v + 6]) * alpha, __uint_as_float(acc[8 * v + 7]) * alpha, p.out_bf16))
                                         : "memory");
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_x, box, col0, tm * BM + quad * 32);
                        tma_store_commit();
                    }
                    sbuf ^= 1;
                }
            } else
#pragma unroll 1
            for (int c = 0; c < bn / 32; c++) {
                const int col0 = n0 + c * 32;
                if (col0 >= p.N) break;  // uniform across the CTA
                uint32_t acc[32];
                tmem_ld_32x32b_x32(taddr + c * 32, acc);
                tmem_ld_wait();
                if (p.X && p.x_tma) {
                    // X += tile through the memory system: own row of the 32 x 32 box into swizzled staging, then one
                    // TMA reduce-add per warp and chunk (rows >= M and columns >= N are clipped by the tensor map)
                    const uint32_t box = staging + (quad * 2 + sbuf) * STAGING_BOX;
                    if (lane == 0) tma_store_wait_read<1>();  // the reduce that used this buffer two chunks ago has read it
                    __syncwarp();
#pragma unroll
                    for (int v = 0; v < 8; v++) {
                        const uint32_t dst = box + lane * 128 + ((v ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(__uint_as_float(acc[4 * v + 0]) * alpha),
                                     "f"(__uint_as_float(acc[4 * v + 1]) * alpha), "f"(__uint_as_float(acc[4 * v + 2]) * alpha),
                                     "f"(__uint_as_float(acc[4 * v + 3]) * alpha)
                                     : "memory");
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_reduce_add_2d(&tmap_x, box, col0, tm * BM + quad * 32);
                        tma_store_commit();
                    }
                    sbuf ^= 1;
                } else if (p.D8) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        v[j] = __uint_as_float(acc[j]) * alpha;
                        tmax = fmaxf(tmax, fabsf(v[j]));
                        v[j] *= scale_d;
                    }
                    if (row < p.M) {
                        uint8_t* drow = p.D8 + (size_t)row * p.N + col0;
                        if (dvec_ok && col0 + 32 <= p.N) {
#pragma unroll
                            for (int h = 0; h < 2; h++) {
                                uint4 o;
                                o.x = pack_e4m3x4(v[16 * h + 0], v[16 * h + 1], v[16 * h + 2], v[16 * h + 3]);
                                o.y = pack_e4m3x4(v[16 * h + 4], v[16 * h + 5], v[16 * h + 6], v[16 * h + 7]);
                                o.z = pack_e4m3x4(v[16 * h + 8], v[16 * h + 9], v[16 * h + 10], v[16 * h + 11]);
                                o.w = pack_e4m3x4(v[16 * h + 12], v[16 * h + 13], v[16 * h + 14], v[16 * h + 15]);
                                __stcs(reinterpret_cast<uint4*>(drow) + h, o);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const uint32_t w = pack_e4m3x4(v[j], v[j + 1], v[j + 2], v[j + 3]);
#pragma unroll
                                for (int e = 0; e < 4; e++)
                                    if (col0 + j + e < p.N) drow[j + e] = (uint8_t)(w >> (8 * e));
                            }
                        }
                    }
                } else if (row < p.M && p.X) {
                    float* xrow = p.X + (size_t)row * p.N + col0;
                    if (xvec_ok && col0 + 32 <= p.N) {
#pragma unroll
                        for (int v = 0; v < 8; v++) {
                            float4 x = *reinterpret_cast<float4*>(xrow + 4 * v);
                            x.x = fmaf(__uint_as_float(acc[4 * v + 0]), alpha, x.x);
                            x.y = fmaf(__uint_as_float(acc[4 * v + 1]), alpha, x.y);
                            x.z = fmaf(__uint_as_float(acc[4 * v + 2]), alpha, x.z);
                            x.w = fmaf(__uint_as_float(acc[4 * v + 3]), alpha, x.w);
                            *reinterpret_cast<float4*>(xrow + 4 * v) = x;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < p.N) xrow[j] = fmaf(__uint_as_float(acc[j]), alpha, xrow[j]);
                    }
                } else if (row < p.M) {
                    if (vec_ok && col0 + 32 <= p.N) {
                        uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            uint4 o;
                            o.x = pack_out(__uint_as_float(acc[8 * v + 0]) * alpha, __uint_as_float(acc[8 * v + 1]) * alpha, p.out_bf16);
                            o.y = pack_out(__uint_as_float(acc[8 * v + 2]) * alpha, __uint_as_float(acc[8 * v + 3]) * alpha, p.out_bf16);
                            o.z = pack_out(__uint_as_float(acc[8 * v + 4]) * alpha, __uint_as_float(acc[8 * v + 5]) * alpha, p.out_bf16);
                            o.w = pack_out(__uint_as_float(acc[8 * v + 6]) * alpha, __uint_as_float(acc[8 * v + 7]) * alpha, p.out_bf16);
                            __stcs(dst + v, o);  // streaming store: C is not read again, keep A and B panels in L2
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            if (col0 + j < p.N) {
                                const float f = __uint_as_float(acc[j]) * alpha;
                                uint16_t bits;
                                if (p.out_bf16) { __nv_bfloat16 h = __float2bfloat16_rn(f); bits = *reinterpret_cast<uint16_t*>(&h); }
                                else { __half h = __float2half_rn(f); bits = *reinterpret_cast<uint16_t*>(&h); }
                                crow[col0 + j] = bits;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
            buf ^= 1;
            if (p.amax) {
                if (row >= p.M) tmax = 0.f;   // rows past M may hold anything when A is loaded with a short box
                // columns past the matrix hold zeros (zero-filled operand rows): they never raise the maximum
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
                if (lane == 0) atomicMax(reinterpret_cast<unsigned int*>(p.amax), __float_as_uint(tmax));
            }
        }
    epilogue_done:
        if (((p.X && p.x_tma) || p.c_tma || p.h_tma || p.d_tma) && lane == 0) tma_store_wait<0>();  // every reduce has left shared memory and been performed
    }

    // ------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    const uint32_t code = *abort_flag;
    if (code != 0) {
        // a wait ran out: report, then give copies already in flight a bounded
        // time to land before shared memory and TMEM are released
        if (threadIdx.x == 0) atomicCAS(&g_gemm_status, 0u, code);
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

__global__ void __launch_bounds__(32) gemm_wait_expiry_selftest_kernel() {
    wait_expiry_selftest_body(&g_gemm_status, ST_TIMEOUT_SELFTEST);
}

// ---------------------------------------------------------------- host side

constexpr int Tile_KSUB(int bn) { return bn == 256 ? Tile<256>::KSUB : bn == 128 ? Tile<128>::KSUB : Tile<64>::KSUB; }

struct DeviceState {
    std::once_flag once;      // first call on this device, from whichever host thread gets there first
    cudaError_t init_error = cudaSuccess;
    int num_sms = 0;
};
constexpr int MAX_DEVICES = 64;
DeviceState g_dev[MAX_DEVICES];

// Tile-pair policy: -1 = choose per problem (default), 0 = never (single tiles only).  The environment variable
// FP8_GEMM_NO_PAIR is read once, at the first launch of the process; fp8_gemm_set_tile_pairs overrides it.
std::atomic<int> g_pair_policy{-2};  // -2 = environment not read yet
int pair_policy() {
    int v = g_pair_policy.load(std::memory_order_acquire);
    if (v == -2) {
        int from_env = getenv("FP8_GEMM_NO_PAIR") ? 0 : -1;
        g_pair_policy.compare_exchange_strong(v, from_env, std::memory_order_acq_rel);
        v = g_pair_policy.load(std::memory_order_acquire);
    }
    return v;
}

void init_device(DeviceState* st, int dev) {
    int major = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) { st->init_error = e; return; }
    if (major != 10) { st->init_error = cudaErrorNoKernelImageForDevice; return; }
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) { st->init_error = e; return; }
    if ((e = cudaFuncSetAttribute(fp8_gemm_tcgen05_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Tile<256>::SMEM_BYTES)) != cudaSuccess) { st->init_error = e; return; }
    if ((e = cudaFuncSetAttribute(fp8_gemm_tcgen05_kernel<256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Tile<256, 2>::SMEM_BYTES)) != cudaSuccess) { st->init_error = e; return; }
    if ((e = cudaFuncSetAttribute(fp8_gemm_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Tile<128>::SMEM_BYTES)) != cudaSuccess) { st->init_error = e; return; }
    if ((e = cudaFuncSetAttribute(fp8_gemm_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Tile<64>::SMEM_BYTES)) != cudaSuccess) { st->init_error = e; return; }
    st->num_sms = sms;
}

int launch(int M, int N, int K, const void* A, const void* B, void* C, float alpha, const float* sa, const float* sb,
           int out_bf16, cudaStream_t stream, float* X = nullptr, void* H = nullptr, int F = 0, float* amax = nullptr,
           uint8_t* D8 = nullptr, const float* scale_d = nullptr) {
    if (M < 0 || N < 0 || K < 0) return (int)cudaErrorInvalidValue;
    if (M == 0 || N == 0) return 0;
    if (!A || !B || (!C && !X && !H && !D8)) return (int)cudaErrorInvalidValue;
    if (H && (!amax || F <= 0 || N != 2 * ((F + 31) / 32) * 32 || (reinterpret_cast<uintptr_t>(H) & 1))) return (int)cudaErrorInvalidValue;
    if (K == 0 || (K % 16) != 0) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
        (reinterpret_cast<uintptr_t>(C) & 1) || (reinterpret_cast<uintptr_t>(X) & 3))
        return (int)cudaErrorInvalidValue;

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    DeviceState& st = g_dev[dev];
    std::call_once(st.once, init_device, &st, dev);
    if (st.init_error != cudaSuccess) return (int)st.init_error;

    // Tile width: 256 unless a narrower tile cuts (waves x per-k-block MMA time) by more than a quarter —
    // i.e. only when the 128x256 tiling leaves most SMs idle (small or skinny problems).  Per-k-block MMA
    // time: 128 / 64 / 48 clocks for BN = 256 / 128 / 64 (the last one limited by operand reads).
    // (For a single row of tiles, choosing the width by the rows of B the busiest SM has to stream instead was
    // measured and is slower: 16 x 32768 x 8192 62 us against 52 us, 64 x 22016 x 4096 26 us against 19 us.)
    const long long m_tiles = (M + BM - 1) / BM;
    auto estimate = [&](int width, int clocks) {
        const long long tiles = m_tiles * ((N + width - 1) / width);
        return ((tiles + st.num_sms - 1) / st.num_sms) * clocks;
    };
    int bn = 256;
    long long best = estimate(256, 128) * 3 / 4;
    if (estimate(128, 64) < best) { best = estimate(128, 64); bn = 128; }
    if (estimate(64, 48) < best) { best = estimate(64, 48); bn = 64; }

    // Tile pairs: with at least two waves of 256 x 256 pairs and a K long enough to amortise the three-stage ring, a
    // CTA holds two vertically adjacent 128 x 256 accumulators (both TMEM buffers) and feeds both from each B tile it
    // loads: 32 KB instead of 48 KB of operands per 128 x 256 x 128 block of MMA work (8192^3: 2739 -> 2965 TFLOP/s).
    // (One wave of pairs is enough when K is long: 4096 x 4096 x 8192 98 us against 106 us; with K = 4096 it is not.)
    // A pair-wave costs two tile-waves at about 0.92 of their time, and pair mode has no half-width last wave, so
    // pairs are taken only when that estimate does not lose to single tiles: a pair count just above a multiple of
    // the SM count (150 pairs on 148 SMs) would pay a whole extra double-cost wave.
    // fp8_gemm_set_tile_pairs(0) or FP8_GEMM_NO_PAIR in the environment keeps single tiles (the parity tests compare
    // the two, bit for bit).
    const long long pairs = ((m_tiles + 1) / 2) * ((N + 255) / 256);
    bool pair = (bn == 256) && K >= 2048 && m_tiles >= 2 && pair_policy() != 0 &&
                (pairs >= 2ll * st.num_sms || (pairs >= st.num_sms && K >= 8192));
    if (pair) {
        const long long tiles1 = m_tiles * ((N + 255) / 256);
        const long long rem1 = tiles1 % st.num_sms;
        // single tiles, in hundredths of a wave; a half-width last wave was measured at about 0.9 of a full one
        const long long single_cost = (tiles1 / st.num_sms) * 100 + (rem1 == 0 ? 0 : (2 * rem1 <= st.num_sms ? 90 : 100));
        const long long pair_cost = ((pairs + st.num_sms - 1) / st.num_sms) * 2 * 92;
        if (pair_cost > single_cost) pair = false;
    }
    GemmParams p;
    p.M = M; p.N = N; p.K = K; p.C = C;
    p.alpha = alpha; p.scale_a = sa; p.scale_b = sb; p.out_bf16 = out_bf16;
    p.X = X;
    p.H = H; p.F = F; p.amax = amax;
    p.D8 = D8; p.scale_d = scale_d;
    p.x_tma = (X && (N % 4) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) ? 1 : 0;
    p.c_tma = (C && !X && !H && !D8 && (N % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
    p.h_tma = (H && bn >= 128 && (F % 8) == 0 && (reinterpret_cast<uintptr_t>(H) & 15) == 0) ? 1 : 0;
    p.d_tma = (D8 && !H && !X && bn >= 128 && (N % 16) == 0 && (reinterpret_cast<uintptr_t>(D8) & 15) == 0) ? 1 : 0;
    p.m_tiles = (int)(pair ? (m_tiles + 1) / 2 : m_tiles);   // rows of tiles, or of tile pairs
    p.n_tiles = (N + bn - 1) / bn;
    p.k_blocks = (K + BK - 1) / BK;

    // The last wave: when the 128x256 tiling leaves it at most half full, its tiles run as two 128x128 units each
    // (same MMA efficiency per flop), so that wave takes half the time instead of idling most SMs.
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles >= (1ll << 30)) return (int)cudaErrorInvalidValue;
    const int rem = (int)(tiles % st.num_sms);
    const bool split_tail = (bn == 256) && !pair && tiles > st.num_sms && rem > 0 && 2 * rem <= st.num_sms;
    p.split_from = (int)(split_tail ? tiles - rem : tiles);
    p.num_units = (int)(split_tail ? tiles + rem : tiles);
    // Split-K: a problem with fewer tiles than half the SMs and a long K (the O and down projections of a decode
    // step: 16 x 4096 x 11008 is 64 tiles) leaves most SMs idle while each busy one streams a long panel of B.
    // Where the result is added into X by TMA reduce anyway, slices of K go to different CTAs and each adds its
    // partial sum (the order of those fp32 additions is then not fixed from run to run).
    const int k_stages = (p.k_blocks + Tile_KSUB(bn) - 1) / Tile_KSUB(bn);
    p.ksplit = 1;
    if (p.x_tma && !split_tail && 2 * tiles <= st.num_sms) {
        long long ks = st.num_sms / tiles;
        if (ks > k_stages / 4) ks = k_stages / 4;   // at least four pipeline stages of work per slice
        if (ks > 8) ks = 8;
        if (ks > 1) p.ksplit = (int)ks;
    }
    p.ks_per = (k_stages + p.ksplit - 1) / p.ksplit;
    p.ksplit = (k_stages + p.ks_per - 1) / p.ks_per;   // no empty slice
    p.num_units *= p.ksplit;

    p.a_rows = BM;
    if (m_tiles == 1 && M <= 64) p.a_rows = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    CUtensorMap ta, tb, tbh;
    if (!make_tmap_u8_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint32_t)p.a_rows, BK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_tmap_u8_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint32_t)bn, BK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_tmap_u8_2d(&tbh, B, (uint64_t)N, (uint64_t)K, (uint32_t)(bn == 256 ? 128 : bn), BK, CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;

    CUtensorMap tx = ta;  // placeholder when there is nothing to describe
    if (p.x_tma && !make_tmap_f32_2d(&tx, X, (uint64_t)M, (uint64_t)N, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return (int)cudaErrorInvalidValue;
    if (p.c_tma && !make_tmap_u16_2d(&tx, C, (uint64_t)M, (uint64_t)N, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return (int)cudaErrorInvalidValue;
    if (p.h_tma && !make_tmap_u16_2d(&tx, H, (uint64_t)M, (uint64_t)F, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return (int)cudaErrorInvalidValue;
    if (p.d_tma && !make_tmap_u8_2d(&tx, D8, (uint64_t)M, (uint64_t)N, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return (int)cudaErrorInvalidValue;

    const int grid = (int)(p.num_units < st.num_sms ? p.num_units : st.num_sms);
    if (pair) fp8_gemm_tcgen05_kernel<256, 2><<<grid, NUM_THREADS, Tile<256, 2>::SMEM_BYTES, stream>>>(ta, tb, tbh, tx, p);
    else if (bn == 256) fp8_gemm_tcgen05_kernel<256><<<grid, NUM_THREADS, Tile<256>::SMEM_BYTES, stream>>>(ta, tb, tbh, tx, p);
    else if (bn == 128) fp8_gemm_tcgen05_kernel<128><<<grid, NUM_THREADS, Tile<128>::SMEM_BYTES, stream>>>(ta, tb, tbh, tx, p);
    else fp8_gemm_tcgen05_kernel<64><<<grid, NUM_THREADS, Tile<64>::SMEM_BYTES, stream>>>(ta, tb, tbh, tx, p);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int fp8_gemm(int M, int N, int K, const void* A, const void* B, void* C, int mode, void* stream) {
    (void)mode;  // 0 and 1 name the reference's two mma.sync variants; one tcgen05 kernel serves both
    return launch(M, N, K, A, B, C, 1.0f, nullptr, nullptr, 0, (cudaStream_t)stream);
}

int fp8_gemm_original(int M, int N, int K, const void* A, const void* B, void* C, void* stream) {
    return fp8_gemm(M, N, K, A, B, C, 0, stream);
}

int fp8_gemm_singlesync(int M, int N, int K, const void* A, const void* B, void* C, void* stream) {
    return fp8_gemm(M, N, K, A, B, C, 1, stream);
}

int fp8_gemm_scaled(int M, int N, int K, const void* A, const void* B, void* C, float alpha, const float* scale_a,
                    const float* scale_b, int out_dtype, void* stream) {
    if (out_dtype != FP8_GEMM_OUT_FP16 && out_dtype != FP8_GEMM_OUT_BF16) return (int)cudaErrorInvalidValue;
    return launch(M, N, K, A, B, C, alpha, scale_a, scale_b, out_dtype == FP8_GEMM_OUT_BF16, (cudaStream_t)stream);
}

int fp8_gemm_accumulate_f32(int M, int N, int K, const void* A, const void* B, float* X, float alpha, const float* scale_a,
                            const float* scale_b, void* stream) {
    if (!X) return (int)cudaErrorInvalidValue;
    return launch(M, N, K, A, B, nullptr, alpha, scale_a, scale_b, 0, (cudaStream_t)stream, X);
}

int fp8_gemm_swiglu(int M, int F, int K, const void* A, const void* B_interleaved, void* H, float alpha, const float* scale_a,
                    const float* scale_b, float* amax_out, void* stream) {
    if (!H || !amax_out || F <= 0) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    const int n = 2 * ((F + 31) / 32) * 32;
    return launch(M, n, K, A, B_interleaved, nullptr, alpha, scale_a, scale_b, 1, (cudaStream_t)stream, nullptr, H, F, amax_out);
}

int fp8_gemm_fp8out(int M, int N, int K, const void* A, const void* B, void* D, float alpha, const float* scale_a,
                    const float* scale_b, const float* scale_d, float* amax_d, void* stream) {
    if (!D) return (int)cudaErrorInvalidValue;
    if (amax_d) {
        cudaError_t e = cudaMemsetAsync(amax_d, 0, sizeof(float), (cudaStream_t)stream);
        if (e != cudaSuccess) return (int)e;
    }
    return launch(M, N, K, A, B, nullptr, alpha, scale_a, scale_b, 0, (cudaStream_t)stream, nullptr, nullptr, 0, amax_d,
                  reinterpret_cast<uint8_t*>(D), scale_d);
}

int fp8_gemm_device_status(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return -(int)e;
    uint32_t code = 0, zero = 0;
    e = cudaMemcpyFromSymbol(&code, g_gemm_status, sizeof(code));
    if (e != cudaSuccess) return -(int)e;
    if (code != 0) cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(zero));
    return (int)code;
}

int fp8_gemm_selftest_wait_expiry(void* stream) {
    gemm_wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
    return (int)cudaGetLastError();
}

int fp8_gemm_set_tile_pairs(int mode) {
    if (mode != 0 && mode != -1) return (int)cudaErrorInvalidValue;
    g_pair_policy.store(mode, std::memory_order_release);
    return 0;
}

const char* fp8_gemm_version(void) { return "1.0.0+tcgen05-sm100a"; }

}  // extern "C"
