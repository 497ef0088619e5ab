// fa_fwd_sm100.cu — FP8 (e4m3) FlashAttention forward for NVIDIA B200 (sm_100a).
//
// Same function as goml's libs/fa_sm120/src/_v121r_train_kernel.cu:208-723 (hd128)
// and libs/flash_attention_v89_pinregs_fp8_forward.cu:201-211 (hd64): per (batch*head),
// O = softmax(scale * Q K^T + mask) V with an online (blockwise) softmax, fp16 output
// and optional natural-log LSE — rebuilt around the Blackwell data path:
//
//   pre-pass       : V (e4m3) -> fp16 copy in a caller-provided workspace (exact:
//                    every e4m3 value is an fp16 value; HBM-bound, <2% of the time)
//   TMA            : swizzled tiles, 3-D maps over [BH,S,D] so a tile never crosses a head
//   S = Q K^T      : tcgen05.mma kind::f8f6f4 on the e4m3 codes, 128x64 fp32
//                    accumulator in TMEM, double buffered so the next block's scores are
//                    ready before the softmax of the current one ends
//   softmax        : 4 warps, one query row per thread (tcgen05.ld 32x32b), fp32 running
//                    max/sum in the log2 domain, scale folded into one packed FFMA per two
//                    scores, lazy O rescale (only when the max grows by more than 2^TAU)
//   P              : kept in fp16 (11-bit significand) and written back to TENSOR MEMORY
//                    over the first half of its S buffer.  The reference rounds P to e4m3 (3-bit
//                    mantissa); for zero-mean V that rounding alone costs ~2.5e-2 mean
//                    relative error, above the 1e-2 bar, so P V runs as an fp16 MMA
//   O += P V       : tcgen05.mma kind::f16, A = P read from TMEM, B = V consumed MN-major
//                    straight from the TMA tile (no shared-memory transpose), fp32
//                    accumulator in TMEM
//   epilogue       : O * (v_descale / l) -> fp16, 128-bit stores; LSE.
//
// The tensor core reads shared-memory operands at 128 B/clk/SM, which is what bounds both
// MMAs here; keeping P out of shared memory keeps that traffic near the exponential-unit
// time, which is the next bound (16 ex2 per clock per SM).  One CTA = one 128-row query tile of one head; 6 warps (4 softmax,
// 1 MMA issuer, 1 TMA producer); two CTAs share an SM so one CTA's softmax overlaps the
// other's MMAs.  Every mbarrier wait is bounded.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <stdio.h>

#include <mutex>

#include "../../include/fa_sm120.h"
#include "fa_fwd_sm100.h"
#include "sm100_ptx.cuh"
#include "tmap.cuh"

namespace fa_sm100 {

using namespace sm100;

namespace {

constexpr int BM = 128;  // query rows per CTA (= TMEM lanes)
constexpr int BN = 64;   // keys per block
constexpr int STAGES = 3; // K / V shared-memory ring depth
constexpr int NUM_SOFTMAX_WARPS = 4;   // one thread per query row
constexpr int HEAD_GROUP = 16;         // heads whose tiles are interleaved when tiles differ in length (48 MB of K/V at S = 8192, D = 128)
constexpr int NUM_THREADS = (NUM_SOFTMAX_WARPS + 2) * 32;
constexpr int MMA_WARP = NUM_SOFTMAX_WARPS;
constexpr int TMA_WARP = NUM_SOFTMAX_WARPS + 1;
constexpr float TAU = 6.0f;   // lazy-rescale threshold (log2 units)
constexpr float POFF = 2.0f;  // P is carried as P * 2^POFF (max 2^(TAU+POFF) = 256, far inside fp16)

enum : uint32_t {
    ST_TIMEOUT_LOAD = 0x201,
    ST_TIMEOUT_MMA = 0x202,
    ST_TIMEOUT_SOFTMAX = 0x203,
    ST_BAD_SMEM_ALIGN = 0x204,
    ST_TIMEOUT_SELFTEST = 0x2F0,   // fa_selftest_wait_expiry
};

__device__ uint32_t g_fa_status = 0;

// Shared memory holds only TMA-written operand tiles.  Both MMAs are limited by how fast the
// tensor core can read its shared-memory operands (128 B/clk/SM), so P never goes through
// shared memory: it is written to tensor memory and read from there as the A operand.
template <int HD>
struct Cfg {
    static constexpr int Q_BYTES = BM * HD;
    static constexpr int K_BYTES = BN * HD;
    static constexpr int V_BYTES = BN * HD * 2;       // fp16
    static constexpr int V_HALF_BYTES = BN * 128;     // one 64-wide (128-byte) slab of d
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V = OFF_K + STAGES * K_BYTES;
    static constexpr int OFF_BAR = OFF_V + STAGES * V_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 256;
    // TMEM: S[0], S[1] (64 fp32 columns each; P of the same block, 32 columns of packed fp16
    //       pairs, overwrites the first half of its S buffer)   O at [128, 128 + HD)
    static constexpr int TMEM_COLS = 256;
    static constexpr int O_COL = 128;
};

struct Params {
    int bh, sl, n_qtiles;
    int causal, window;
    float scale_log2;  // scale * log2(e)
    float v_descale;
    const float* sq;   // optional device scalars (quantiser outputs)
    const float* sk;
    const float* sv;
    __half* o;
    float* lse;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Packed fp32 pairs (Blackwell fma.rn.f32x2 / add.f32x2): one issue slot for two results.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1) {
    asm("{\n\t.reg .b64 ra, rd;\n\t"
        "mov.b64 rd, {%0, %1};\n\tmov.b64 ra, {%2, %3};\n\t"
        "add.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1)
        : "f"(a0), "f"(a1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(32) fa_wait_expiry_selftest_kernel() {
    wait_expiry_selftest_body(&g_fa_status, ST_TIMEOUT_SELFTEST);
}

// V (e4m3) -> fp16, 16 codes per thread per step; exact.
__global__ void __launch_bounds__(256) v_to_f16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, size_t n16) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint4 c = __ldg(in + i);
        const uint32_t w[4] = {c.x, c.y, c.z, c.w};
        uint32_t h[8];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h[2 * k]) : "h"((uint16_t)(w[k] & 0xffffu)));
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h[2 * k + 1]) : "h"((uint16_t)(w[k] >> 16)));
        }
        out[2 * i] = make_uint4(h[0], h[1], h[2], h[3]);
        out[2 * i + 1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
}

// Sign flip of one row of raw scores for a negative scale (the row max is taken on sign-adjusted scores).
// Rare, so it is kept out of line: the common path pays one not-taken branch instead of 64 predicated ops.
__device__ __noinline__ void negate_scores(uint32_t* s) {
    for (int c = 0; c < BN; c++) s[c] ^= 0x80000000u;
}

// MASKED = false: no key of the launch is masked (non-causal, no window, S a multiple of the block) and the host-side scale
// is positive: neither the masking code nor the sign flip of a negative scale is compiled into the softmax loop.  (The
// device-side scale factors are quantiser outputs, amax / 448: never negative.)
template <int HD, bool MASKED>
__global__ void __launch_bounds__(NUM_THREADS, 2)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const Params p) {
    using C = Cfg<HD>;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + C::OFF_BAR;
    // Completion barriers are indexed by ring stage (block j -> j % STAGES) and double as the
    // "stage free" signals of the K and V rings: one tcgen05.commit per MMA batch instead of two.
    const uint32_t bar_q = bars;
    const uint32_t bar_kfull = bars + 8;                  // [STAGES] K tile landed
    const uint32_t bar_vfull = bar_kfull + 8 * STAGES;    // [STAGES] V tile landed
    const uint32_t bar_sfull = bar_vfull + 8 * STAGES;    // [STAGES] S = Q K^T of that block complete (K stage reusable)
    const uint32_t bar_pvdone = bar_sfull + 8 * STAGES;   // [STAGES] O += P V of that block complete (V stage reusable)
    const uint32_t bar_pfull = bar_pvdone + 8 * STAGES;   // [2] softmax wrote P into S[b] (and rescaled O if needed)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 240);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;

    // tile -> (head, query tile).  Tiles of equal cost go head by head, so that the CTAs in
    // flight share a few heads' K/V in L2.  When the key range depends on the query tile
    // (causal, window) the heads are taken in groups of HEAD_GROUP, and inside a group the
    // tiles with the most keys come first across all its heads: the last CTAs of the launch
    // are then the short tiles of a whole group, not the long tiles of the last head.
    int head, qt;
    if (p.causal || p.window > 0) {
        const int per_group = HEAD_GROUP * p.n_qtiles;
        const int g = blockIdx.x / per_group;
        const int r = blockIdx.x - g * per_group;
        const int heads_here = min(HEAD_GROUP, p.bh - g * HEAD_GROUP);
        head = g * HEAD_GROUP + r % heads_here;
        qt = p.n_qtiles - 1 - r / heads_here;
    } else {
        head = blockIdx.x / p.n_qtiles;
        qt = p.n_qtiles - 1 - (blockIdx.x % p.n_qtiles);
    }
    const int q0 = qt * BM;
    // keys this tile can see: [kv_lo, kv_hi)
    const int kv_hi = p.causal ? min(p.sl, q0 + BM) : p.sl;
    const int kv_lo = (p.window > 0) ? max(0, q0 - p.window + 1) : 0;
    const int blk0 = kv_lo / BN;
    const int nblk = (kv_hi + BN - 1) / BN - blk0;  // >= 1

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_kfull + 8 * s, 1);
            mbar_init(bar_vfull + 8 * s, 1);
            mbar_init(bar_sfull + 8 * s, 1);
            mbar_init(bar_pvdone + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) mbar_init(bar_pfull + 8 * b, NUM_SOFTMAX_WARPS * 32);
        *abort_flag = (sbase & 1023u) ? ST_BAD_SMEM_ALIGN : 0u;
        fence_mbar_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;
    const uint32_t tmem_o = tmem_base + C::O_COL;
    const bool bad_start = (*abort_flag != 0);

    if (bad_start) {
        // fall through to teardown
    } else if (warp == TMA_WARP) {
        // ------------------------------------------------------------- TMA producer
        // The whole warp runs the loop and one elected lane issues: addresses and coordinates stay warp-uniform.
        {
            const bool leader = elect_one();
            if (leader) {
                prefetch_tmap(&tmap_q);
                prefetch_tmap(&tmap_k);
                prefetch_tmap(&tmap_v);
                mbar_arrive_expect_tx(bar_q, C::Q_BYTES);
                tma_load_3d(sbase + C::OFF_Q, &tmap_q, bar_q, 0, q0, head);
            }
            int s = 0;
            uint32_t ph = 1;  // "previous phase complete": the rings start empty
            for (int j = 0; j < nblk; j++) {
                const int key0 = (blk0 + j) * BN;
                if (!mbar_wait(bar_sfull + 8 * s, ph, abort_flag, ST_TIMEOUT_LOAD)) break;   // Q K^T three blocks back is done
                if (leader) {
                    mbar_arrive_expect_tx(bar_kfull + 8 * s, C::K_BYTES);
                    tma_load_3d(sbase + C::OFF_K + s * C::K_BYTES, &tmap_k, bar_kfull + 8 * s, 0, key0, head);
                }
                if (!mbar_wait(bar_pvdone + 8 * s, ph, abort_flag, ST_TIMEOUT_LOAD)) break;  // P V three blocks back is done
                if (leader) {
                    mbar_arrive_expect_tx(bar_vfull + 8 * s, C::V_BYTES);
#pragma unroll
                    for (int h = 0; h < HD / 64; h++)  // one 64-column (128-byte) slab of d per copy
                        tma_load_3d(sbase + C::OFF_V + s * C::V_BYTES + h * C::V_HALF_BYTES, &tmap_v, bar_vfull + 8 * s,
                                    h * 64, key0, head);
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == MMA_WARP) {
        // -------------------------------------------------------------- MMA issuer
        // Whole warp, one elected lane issues (descriptors stay in uniform registers).
        {
            const bool leader = elect_one();
            constexpr uint32_t idesc_qk = make_idesc_e4m3_f32(BM, BN, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16_f32(BM, HD, 0, 1);  // A = P from TMEM, V is MN-major
            auto qk_desc = [&](uint32_t addr) { return HD == 128 ? kmajor_desc_sw128(addr) : kmajor_desc_sw64(addr); };
            // K ring position of the next Q K^T, V ring position of the next P V
            int ks = 0, vs = 0;
            uint32_t kph = 0, vph = 0;
            bool ok = true;
            auto issue_qk = [&](int j) {  // S[j & 1] = Q K(j)^T
                ok = mbar_wait(bar_kfull + 8 * ks, kph, abort_flag, ST_TIMEOUT_MMA);
                if (!ok) return;
                tc_fence_after();
                const uint64_t qd = qk_desc(sbase + C::OFF_Q);
                const uint64_t kd = qk_desc(sbase + C::OFF_K + ks * C::K_BYTES);
                if (leader) {
#pragma unroll
                    for (int k = 0; k < HD / 32; k++)
                        mma_f8f6f4_ss(tmem_s + (j & 1) * BN, qd + 2 * k, kd + 2 * k, idesc_qk, k != 0);
                    mma_commit(bar_sfull + 8 * ks);
                }
                __syncwarp();
                if (++ks == STAGES) { ks = 0; kph ^= 1; }
            };
            ok = mbar_wait(bar_q, 0, abort_flag, ST_TIMEOUT_MMA);
            for (int j = 0; j < 2 && j < nblk && ok; j++) issue_qk(j);
            for (int j = 0; j < nblk && ok; j++) {
                const int b = j & 1;
                ok = mbar_wait(bar_vfull + 8 * vs, vph, abort_flag, ST_TIMEOUT_MMA) &&
                     mbar_wait(bar_pfull + 8 * b, (j >> 1) & 1, abort_flag, ST_TIMEOUT_MMA);
                if (!ok) break;
                tc_fence_after();
                const uint32_t vaddr = sbase + C::OFF_V + vs * C::V_BYTES;
                if (leader) {
#pragma unroll
                    for (int k = 0; k < BN / 16; k++) {  // 16 keys per MMA: 8 TMEM columns of P, 16 rows of V
                        const uint64_t vd = mnmajor_desc_sw128(vaddr + k * 16 * 128, C::V_HALF_BYTES);
                        mma_f16_ts(tmem_o, tmem_s + b * BN + 8 * k, vd, idesc_pv, (j | k) != 0);
                    }
                    mma_commit(bar_pvdone + 8 * vs);
                }
                __syncwarp();
                if (++vs == STAGES) { vs = 0; vph ^= 1; }
                // S[b] is rewritten by the Q K^T two blocks ahead; it is issued behind this P V on the
                // same in-order tensor pipe, so P(j) has been read before S(j+2) lands on it
                if (j + 2 < nblk) issue_qk(j + 2);
            }
        }
    } else {
        // ------------------------------------------- softmax / correction / epilogue
        const int r = threadIdx.x;               // row of the tile = TMEM lane (one thread per row)
        const int qi = q0 + r;                   // query index in the sequence
        const uint32_t lane_off = uint32_t(warp * 32) << 16;
        float scale_log2 = p.scale_log2;
        if (p.sq) scale_log2 *= __ldg(p.sq);
        if (p.sk) scale_log2 *= __ldg(p.sk);
        const bool neg = scale_log2 < 0.f;       // the row max is taken on sign-adjusted raw scores
        float ascale = fabsf(scale_log2);
        if (ascale == 0.f) ascale = 1e-30f;      // keeps -inf * scale = -inf for masked keys
        float m_ref = -INFINITY;                 // reference max used in the exponent (log2 units)
        float m_thr = -INFINITY;                 // m_ref + TAU
        float nmsub = 0.f;                       // POFF - m_ref (0 while no finite score has been seen)
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;   // running sum of P * 2^POFF, in four partial sums
        bool ok = true;
        int rs = 0;           // ring stage of block j (j % STAGES) and its phase; those of block j-1
        uint32_t rph = 0;
        int rs_prev = 0;
        uint32_t rph_prev = 0;
        const int hi_key = p.causal ? min(qi, p.sl - 1) : p.sl - 1;   // last visible key of this row
        const int lo_key = (p.window > 0) ? qi - p.window + 1 : 0;    // first visible key

        // Blocks that need per-element masking (uniform across the CTA): those that reach past the sequence end or past the
        // tile's first query (causal) — from j_mask_hi on — and those that start before the window of the tile's last query
        // — below j_mask_lo.  With 64-key blocks and 128-query tiles: (blk0 + j + 1) * BN > sl  <=>  j >= sl / BN - blk0;
        // (blk0 + j + 1) * BN - 1 > q0  <=>  j >= q0 / BN - blk0;  (blk0 + j) * BN < q0 + BM - window  <=>  j < ceil(..) - blk0.
        int j_mask_hi = p.sl / BN - blk0;
        if (p.causal) j_mask_hi = min(j_mask_hi, q0 / BN - blk0);
        const int j_mask_lo = (p.window > 0 && q0 + BM - p.window > 0) ? (q0 + BM - p.window + BN - 1) / BN - blk0 : 0;

        // two blocks per trip: the S buffer index (j & 1) and everything derived from it become compile-time constants
#pragma unroll 2
        for (int j = 0; j < nblk; j++) {
            const int key0 = (blk0 + j) * BN;
            const int b = j & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * rs, rph, abort_flag, ST_TIMEOUT_SOFTMAX))) { ok = false; break; }
            tc_fence_after();
            uint32_t sreg[BN];
#pragma unroll
            for (int c = 0; c < BN / 32; c++) tmem_ld_32x32b_x32(tmem_s + lane_off + b * BN + c * 32, sreg + c * 32);
            tmem_ld_wait();

            if (MASKED && neg) {  // out of line, on a local copy so that sreg stays in registers
                uint32_t tmp[BN];
#pragma unroll
                for (int c = 0; c < BN; c++) tmp[c] = sreg[c];
                negate_scores(tmp);
#pragma unroll
                for (int c = 0; c < BN; c++) sreg[c] = tmp[c];
            }
            // does this block need per-element masking?  (uniform across the CTA)
            const bool mask_blk = MASKED && (j < j_mask_lo || j >= j_mask_hi);
            if (mask_blk) {
                // the empty volatile statement keeps this a real (in the common case not-taken) branch
                // instead of 64 predicated selects executed for every block
                asm volatile("" ::: "memory");
#pragma unroll
                for (int c = 0; c < BN; c++) {
                    const int key = key0 + c;
                    if (key > hi_key || key < lo_key) sreg[c] = 0xff800000u;  // -inf
                }
            }
            float mxa[8];  // eight short dependency chains
#pragma unroll
            for (int t = 0; t < 8; t++) mxa[t] = fmaxf(__uint_as_float(sreg[2 * t]), __uint_as_float(sreg[2 * t + 1]));
#pragma unroll
            for (int c = 16; c < BN; c += 16) {
#pragma unroll
                for (int t = 0; t < 8; t++)
                    mxa[t] = max3(mxa[t], __uint_as_float(sreg[c + 2 * t]), __uint_as_float(sreg[c + 2 * t + 1]));
            }
            const float mx = fmaxf(max3(max3(mxa[0], mxa[1], mxa[2]), max3(mxa[3], mxa[4], mxa[5]), mxa[6]), mxa[7]) * ascale;

            // The reference moves only when some row's maximum exceeds it by more than 2^TAU (always on the first finite
            // maximum: m_thr starts at -inf); everything that depends on it is state updated in this rare branch, so the
            // common path is one compare and one vote.
            if (__any_sync(0xffffffffu, mx > m_thr)) {
                const bool bump = mx > m_thr;
                const float m_new = bump ? mx : m_ref;
                if (j > 0) {
                    // O is final only once the previous P V has finished
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_pvdone + 8 * rs_prev, rph_prev, abort_flag, ST_TIMEOUT_SOFTMAX))) { ok = false; break; }
                    tc_fence_after();
                    const float f = bump ? ex2(m_ref - m_new) : 1.0f;  // m_ref = -inf -> 0
                    l0 *= f; l1 *= f; l2 *= f; l3 *= f;
#pragma unroll
                    for (int c = 0; c < HD / 16; c++) {
                        uint32_t o[16];
                        tmem_ld_32x32b_x16(tmem_o + lane_off + c * 16, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st_32x32b_x16(tmem_o + lane_off + c * 16, o);
                    }
                }
                m_ref = m_new;
                m_thr = m_ref + TAU;
                nmsub = (m_ref == -INFINITY) ? 0.f : POFF - m_ref;
            }

#pragma unroll
            for (int g = 0; g < BN / 32; g++) {  // 32 keys -> 16 TMEM columns of packed fp16 pairs
                uint32_t w[16];
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    float x0, x1;
                    ffma2(x0, x1, __uint_as_float(sreg[g * 32 + q * 2 + 0]), __uint_as_float(sreg[g * 32 + q * 2 + 1]),
                          ascale, ascale, nmsub, nmsub);
                    const float p0 = ex2(x0);
                    const float p1 = ex2(x1);
                    if (q & 1) fadd2(l2, l3, p0, p1); else fadd2(l0, l1, p0, p1);
                    w[q] = pack_half2(p0, p1);
                }
                tmem_st_32x32b_x16(tmem_s + lane_off + b * BN + g * 16, w);  // P overwrites the first half of S[b]
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_pfull + 8 * b);
            rs_prev = rs;
            rph_prev = rph;
            if (++rs == STAGES) { rs = 0; rph ^= 1; }
        }

        // epilogue: O / l (times the V dequantisation scale) -> fp16
        if (ok && __all_sync(0xffffffffu, mbar_wait(bar_pvdone + 8 * rs_prev, rph_prev, abort_flag, ST_TIMEOUT_SOFTMAX))) {
            tc_fence_after();
            const float l = (l0 + l1) + (l2 + l3);
            const float vds = p.sv ? p.v_descale * __ldg(p.sv) : p.v_descale;
            const float inv = (l > 0.f) ? vds / l : 0.f;
            // O leaves through shared memory so that the global stores are coalesced: a thread owns one row (HD fp16 = ROWB
            // bytes), which written straight to global makes every store instruction of a warp touch 32 different lines.
            // Each warp stages its 32 rows in the (by now idle) K ring — 16-byte chunk c of row r at chunk c ^ (r % CPR), so
            // that both the row-wise writes and the read-back are free of bank conflicts — and stores them back as whole
            // 512-byte runs.  Only this warp touches its staging area: a __syncwarp() orders the two passes.
            constexpr int ROWB = HD * 2;            // bytes per output row
            constexpr int CPR = ROWB / 16;          // 16-byte chunks per row: 16 (D = 128) or 8 (D = 64)
            uint8_t* stage = smem + C::OFF_K + warp * (32 * ROWB);
            const int lane = threadIdx.x & 31;
#pragma unroll
            for (int c = 0; c < HD / 16; c++) {
                uint32_t o[16];
                tmem_ld_32x32b_x16(tmem_o + lane_off + c * 16, o);
                tmem_ld_wait();
#pragma unroll
                for (int v = 0; v < 2; v++) {
                    uint4 w;
                    w.x = pack_half2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                    w.y = pack_half2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                    w.z = pack_half2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                    w.w = pack_half2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                    const int ch = 2 * c + v;
                    *reinterpret_cast<uint4*>(stage + lane * ROWB + ((ch ^ (lane % CPR)) << 4)) = w;
                }
            }
            __syncwarp();
            {
                constexpr int RPI = 32 / CPR;       // rows per store instruction: 2 (D = 128) or 4 (D = 64)
                uint8_t* obase = reinterpret_cast<uint8_t*>(p.o + ((size_t)head * p.sl + q0 + warp * 32) * HD);
                const int rows_left = p.sl - (q0 + warp * 32);   // rows of this warp inside the sequence
#pragma unroll
                for (int i = 0; i < 32 / RPI; i++) {
                    const int rr = i * RPI + lane / CPR, ch = lane % CPR;
                    const uint4 w = *reinterpret_cast<const uint4*>(stage + rr * ROWB + ((ch ^ (rr % CPR)) << 4));
                    if (rr < rows_left) *reinterpret_cast<uint4*>(obase + (size_t)rr * ROWB + (ch << 4)) = w;
                }
            }
            if (p.lse && qi < p.sl) {
                // sum_j exp(s_j) = l * 2^(m_ref - POFF)  ->  natural-log LSE
                p.lse[(size_t)head * p.sl + qi] =
                    (l > 0.f) ? (m_ref - POFF + log2f(l)) * 0.6931471805599453f : -INFINITY;
            }
        }
    }

    // ----------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    const uint32_t code = *abort_flag;
    if (code != 0) {
        if (threadIdx.x == 0) atomicCAS(&g_fa_status, 0u, code);
        for (int i = 0; i < 200; i++) __nanosleep(1000);  // let copies already in flight land
        __syncthreads();
    }
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

struct DeviceState {
    std::once_flag once;   // first call on this device, from whichever host thread gets there first
    cudaError_t init_error = cudaSuccess;
    int num_sms = 148;
};
DeviceState g_dev[64];

void init_device(DeviceState* st, int dev);

template <int HD>
cudaError_t launch_hd(const LaunchArgs& a, int num_sms) {
    using C = Cfg<HD>;
    const size_t n = (size_t)a.bh * a.sl * HD;
    // pre-pass: V codes -> fp16 workspace
    {
        const size_t n16 = n / 16;  // HD is a multiple of 16
        size_t blocks = (n16 + 255) / 256;
        const size_t cap = (size_t)num_sms * 8;
        if (blocks > cap) blocks = cap;
        v_to_f16_kernel<<<(unsigned)blocks, 256, 0, a.stream>>>(reinterpret_cast<const uint4*>(a.v),
                                                               reinterpret_cast<uint4*>(a.v16_workspace), n16);
    }
    CUtensorMap tq, tk, tv;
    const CUtensorMapSwizzle swz = (HD == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    if (!make_tmap_u8_3d(&tq, a.q, a.bh, a.sl, HD, BM, HD, swz) ||
        !make_tmap_u8_3d(&tk, a.k, a.bh, a.sl, HD, BN, HD, swz) ||
        !make_tmap_u16_3d(&tv, a.v16_workspace, a.bh, a.sl, HD, BN, 64, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    Params p;
    p.bh = a.bh; p.sl = a.sl; p.n_qtiles = (a.sl + BM - 1) / BM;
    p.causal = a.causal; p.window = a.window;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.v_descale = a.v_descale;
    p.sq = a.scale_q_dev; p.sk = a.scale_k_dev; p.sv = a.scale_v_dev;
    p.o = reinterpret_cast<__half*>(a.o);
    p.lse = a.lse;
    const long long grid = (long long)a.bh * p.n_qtiles;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    const bool masked = a.causal || a.window > 0 || (a.sl % BN) != 0 || !(a.scale > 0.f);
    if (masked) fa_fwd_kernel<HD, true><<<(unsigned)grid, NUM_THREADS, C::SMEM_BYTES, a.stream>>>(tq, tk, tv, p);
    else fa_fwd_kernel<HD, false><<<(unsigned)grid, NUM_THREADS, C::SMEM_BYTES, a.stream>>>(tq, tk, tv, p);
    return cudaGetLastError();
}

}  // namespace

namespace {
void init_device(DeviceState* st, int dev) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fwd_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fwd_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<64>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fwd_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<64>::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&st->num_sms, cudaDevAttrMultiProcessorCount, dev);
    st->init_error = e;
}
}  // namespace

size_t workspace_bytes(int bh, int sl, int hd) { return (size_t)bh * sl * hd * 2; }

cudaError_t launch(const LaunchArgs& a) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!a.v16_workspace || (reinterpret_cast<uintptr_t>(a.v16_workspace) & 127)) return cudaErrorInvalidValue;
    std::call_once(g_dev[dev].once, init_device, &g_dev[dev], dev);
    if (g_dev[dev].init_error != cudaSuccess) return g_dev[dev].init_error;
    return a.hd == 128 ? launch_hd<128>(a, g_dev[dev].num_sms) : launch_hd<64>(a, g_dev[dev].num_sms);
}

cudaError_t launch_wait_expiry_selftest(cudaStream_t stream) {
    fa_wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>();
    return cudaGetLastError();
}

int device_status() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return -(int)e;
    uint32_t code = 0, zero = 0;
    e = cudaMemcpyFromSymbol(&code, g_fa_status, sizeof(code));
    if (e != cudaSuccess) return -(int)e;
    if (code != 0) cudaMemcpyToSymbol(g_fa_status, &zero, sizeof(zero));
    return (int)code;
}

// ----------------------------------------------------------------------------------------
// Forward pass for callers that must not allocate.
//
// The regular entry points borrow their scratch (the fp16 copy of V) from a memory pool.
// Some callers cannot do that: code embedded in a framework that reserved the whole GPU up
// front and forbids any later cudaMalloc-family call, and real-time or safety-certified
// processes whose device memory map is frozen after start-up.  For them the scratch lives in
// the fixed device array below, which every GPU that loads this library carries until the
// process exits (32 MiB).  That caps one call at FA_NOALLOC_MAX_ELEMS elements of V.
//
// The array is shared by every call on that GPU and keeps the previous call's contents.
// Nothing in it has to start at zero: the pre-pass rewrites every element the kernel will read
// before the kernel runs.  Two calls whose GPU work overlaps (different streams) race on it;
// issue them on one stream or serialise them.  The first call on each device also looks up the
// array's device address and sets kernel attributes; make that first call before starting any
// stream capture.
// ----------------------------------------------------------------------------------------
constexpr size_t FA_NOALLOC_MAX_ELEMS = (size_t)16 << 20;  // batch_heads * seq_len * head_dim <= 16 Mi
static __device__ __align__(256) uint16_t g_noalloc_v16[FA_NOALLOC_MAX_ELEMS];

namespace {
// In host code `g_noalloc_v16` is only a stand-in for the device array; the device address is
// looked up once per device (with that device current) and cached.
struct NoallocState {
    std::once_flag once;
    fa_status_t status = FA_OK;
    cudaError_t cuda_error = cudaSuccess;
    void* ptr = nullptr;
};
NoallocState g_noalloc[64];

// One-time set-up for a device, run with that device current (do it before any stream capture): architecture
// check and the device address of the scratch array.  With lazy module loading this is also where the driver
// reserves the array's 32 MiB on that GPU.
void noalloc_init(NoallocState* st, int dev) {
    int major = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) { st->status = FA_ERR_CUDA; st->cuda_error = e; return; }
    if (major != 10) { st->status = FA_ERR_UNSUPPORTED_ARCH; return; }
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_v16);
    if (e != cudaSuccess || !ptr) { st->status = FA_ERR_CUDA; st->cuda_error = e; return; }
    st->ptr = ptr;
}

void write_msg(char* err, int err_len, const char* msg) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", msg);
}
}  // namespace

}  // namespace fa_sm100

extern "C" __attribute__((visibility("default")))
fa_status_t fa_forward_noalloc(const fa_forward_args_t* g, char* err, int err_len) {
    using namespace fa_sm100;
    if (err && err_len > 0) err[0] = '\0';
    if (!g) { write_msg(err, err_len, "fa_forward_noalloc: null argument block"); return FA_ERR_INVALID_ARG; }
    if (!g->q || !g->k || !g->v || !g->o) { write_msg(err, err_len, "fa_forward_noalloc: null pointer in q/k/v/o"); return FA_ERR_INVALID_ARG; }
    if (g->batch_heads <= 0 || g->seq_len <= 0) { write_msg(err, err_len, "fa_forward_noalloc: bh/sl must be > 0"); return FA_ERR_INVALID_ARG; }
    if (g->head_dim != 64 && g->head_dim != 128) { write_msg(err, err_len, "fa_forward_noalloc: head_dim must be 64 or 128"); return FA_ERR_UNSUPPORTED_HD; }
    if (g->window < 0 || g->window > g->seq_len) { write_msg(err, err_len, "fa_forward_noalloc: window must be in [0, seq_len]"); return FA_ERR_INVALID_ARG; }
    if (g->causal != 0 && g->causal != 1) { write_msg(err, err_len, "fa_forward_noalloc: causal must be 0 or 1"); return FA_ERR_INVALID_ARG; }
    const uintptr_t align_or = reinterpret_cast<uintptr_t>(g->q) | reinterpret_cast<uintptr_t>(g->k) |
                               reinterpret_cast<uintptr_t>(g->v) | reinterpret_cast<uintptr_t>(g->o);
    if (align_or & 15) { write_msg(err, err_len, "fa_forward_noalloc: q/k/v/o must be 16-byte aligned"); return FA_ERR_INVALID_ARG; }
    if (reinterpret_cast<uintptr_t>(g->l_out) & 3) { write_msg(err, err_len, "fa_forward_noalloc: l_out must be 4-byte aligned"); return FA_ERR_INVALID_ARG; }
    const size_t elems = (size_t)g->batch_heads * (size_t)g->seq_len * (size_t)g->head_dim;
    if (elems > FA_NOALLOC_MAX_ELEMS) {
        if (err && err_len > 0)
            snprintf(err, (size_t)err_len,
                     "fa_forward_noalloc: batch_heads*seq_len*head_dim = %zu exceeds the fixed scratch of %zu elements "
                     "(32 MiB); split the batch or use fa_forward_ex", elems, FA_NOALLOC_MAX_ELEMS);
        return FA_ERR_UNSUPPORTED_SHAPE;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) { write_msg(err, err_len, "fa_forward_noalloc: cudaGetDevice failed"); return FA_ERR_CUDA; }
    NoallocState& st = g_noalloc[dev];
    std::call_once(st.once, noalloc_init, &st, dev);
    if (st.status == FA_ERR_UNSUPPORTED_ARCH) { write_msg(err, err_len, "fa_forward_noalloc: GPU is not compute capability 10.x"); return st.status; }
    if (st.status != FA_OK) {
        if (err && err_len > 0) snprintf(err, (size_t)err_len, "fa_forward_noalloc: set-up (cudaGetSymbolAddress): %s", cudaGetErrorString(st.cuda_error));
        return st.status;
    }
    // same dispatcher consultation as the other entries, so FA_SM120_DEBUG traces every forward call alike
    if (fa_dispatch_select(g->batch_heads, g->seq_len, g->head_dim, g->causal, g->window) == FA_KERNEL_NONE) {
        write_msg(err, err_len, "fa_forward_noalloc: no kernel matches this configuration");
        return FA_ERR_UNSUPPORTED_SHAPE;
    }
    LaunchArgs a{};
    a.q = g->q; a.k = g->k; a.v = g->v; a.o = g->o; a.lse = static_cast<float*>(g->l_out);
    a.bh = g->batch_heads; a.sl = g->seq_len; a.hd = g->head_dim; a.causal = g->causal; a.window = g->window;
    a.scale = g->scale; a.v_descale = (g->v_descale == 0.0f) ? 1.0f : g->v_descale;
    a.scale_q_dev = g->scale_q_dev; a.scale_k_dev = g->scale_k_dev; a.scale_v_dev = g->scale_v_dev;
    a.v16_workspace = st.ptr;
    a.stream = reinterpret_cast<cudaStream_t>(g->stream);
    e = launch(a);
    if (e != cudaSuccess) {
        if (err && err_len > 0) snprintf(err, (size_t)err_len, "fa_forward_noalloc: launch: %s", cudaGetErrorString(e));
        return FA_ERR_CUDA;
    }
    return FA_OK;
}

// Context-free twin of fa_device_status for callers of fa_forward_noalloc, which have no fa_ctx_t (creating one
// would create a memory pool, the very thing they avoid).  Synchronises the current device; allocates nothing.
extern "C" __attribute__((visibility("default")))
int fa_noalloc_device_status(void) { return fa_sm100::device_status(); }
