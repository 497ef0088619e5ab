// fa_decode_sm100.cu — FP8 attention for one new token per sequence against an FP8 KV cache
// (decode step), grouped-query heads, for NVIDIA B200 (sm_100a).
//
//   q        [B, Hq, D]          e4m3   (one token per sequence)
//   k_cache  [B, Hkv, Smax, D]   e4m3   (the layout the prefill kernels read: BH = B*Hkv, S = Smax)
//   v_cache  [B, Hkv, Smax, D]   e4m3
//   o        [B, Hq, D]          fp16,  lse [B, Hq] fp32 (natural log, optional)
//   seq_lens [B] int32 on the device (keys [0, seq_lens[b]) of sequence b are visible), or one length for all
//
// The step reads every cached key and value once and does 4*Hq*D FLOP per key: HBM-bound, so this is a
// streaming kernel, not a tcgen05 one.  One CTA (4 warps) per (sequence, kv head, split of the key range); the
// G = Hq/Hkv (<= 16) query heads that share a kv head form the 16 rows of the warp-level MMAs:
//   S = Q K^T   mma.sync m16n8k32 e4m3 x e4m3 -> fp32, K fragments straight from a padded shared-memory copy
//   P V         mma.sync m16n8k16 fp16 x fp16 -> fp32, P kept in fp16 (an e4m3 P costs 2.5e-2 relative error),
//               V converted to fp16 on its way into shared memory and read with ldmatrix.trans
// Each warp owns 16 of the 64 keys of a chunk and carries its own online-softmax state (m, l, O) over all chunks,
// loading and converting its own keys, so the loop needs only warp-level synchronisation; the four states are merged
// once at the end.  K and V chunks arrive through a 2-stage cp.async ring (one chunk = 16 KB in flight per CTA,
// four CTAs = 16 warps per SM: the loop is bound by instruction issue and dependency stalls, which more warps hide
// better than a deeper ring).  With more than one
// split the partial states go to a workspace and a second kernel merges them.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "fa_fwd_sm100.h"

namespace fa_sm100 {

namespace {

constexpr int CHUNK = 64;     // keys per step of a CTA
constexpr int THREADS = 128;  // 4 warps x 16 keys
constexpr int ROWS = 16;      // MMA rows = query heads of one kv head (padded)
#ifndef FA_DECODE_STAGES
#define FA_DECODE_STAGES 2
#endif
#ifndef FA_DECODE_CTAS
#define FA_DECODE_CTAS 4
#endif
constexpr int STAGES = FA_DECODE_STAGES;     // cp.async ring depth (chunks)
constexpr int CTAS_PER_SM = FA_DECODE_CTAS;  // resident CTAs the register budget is set for

// D = A B with a zero accumulator input (no registers to clear first)
__device__ __forceinline__ void mma_e4m3_m16n8k32_zero(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_f16_m16n8k16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(saddr));
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
struct DecodeParams {
    const uint8_t* q;
    const uint8_t* k;
    const uint8_t* v;
    __half* o;
    float* lse;
    const int* seq_lens;
    int batch, hq, hkv, group, s_max, seq_len;
    float scale_log2, v_descale;
    const float* sq;
    const float* sk;
    const float* sv;
    int splits, chunks_per_split;
    // paged cache: k, v are [num_pages, Hkv, page_size, D]; logical chunk c of sequence b lives in page
    // block_table[b * max_pages + c / chunks_per_page]
    const int* block_table;
    int page_size, max_pages, num_pages, chunks_per_page;
    float* ws_o;   // [B*Hkv, splits, ROWS, D] un-normalised partial outputs
    float* ws_ml;  // [B*Hkv, splits, ROWS, 2] (m in log2 units, l)
};

template <int D>
struct Smem {
    static constexpr int K_STRIDE = D + 16;          // bytes per key row of the e4m3 K copy (16 spreads rows over banks)
    static constexpr int V_STRIDE = 2 * D + 16;      // bytes per key row of the fp16 V copy
    static constexpr int K_BYTES = CHUNK * K_STRIDE;      // one ring stage of K
    static constexpr int VRAW_BYTES = CHUNK * D;          // one ring stage of V codes (dense)
    static constexpr int V_BYTES = CHUNK * V_STRIDE;      // the fp16 copy of the chunk being computed
    static constexpr int OFF_VRAW = STAGES * K_BYTES;
    static constexpr int OFF_V = OFF_VRAW + STAGES * VRAW_BYTES;
    static constexpr int MERGE_BYTES = 4 * ROWS * (D + 2) * 4;   // four warps' (O, m, l) for the final merge
    static constexpr int BYTES = (OFF_V + V_BYTES) > MERGE_BYTES ? (OFF_V + V_BYTES) : MERGE_BYTES;
};

template <int D, bool PAGED>
__global__ void __launch_bounds__(THREADS, CTAS_PER_SM) fa_decode_kernel(const DecodeParams p) {
    using S = Smem<D>;
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* Vs = smem + S::OFF_V;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;              // MMA fragment coordinates
    const int bh = blockIdx.x;                          // sequence * Hkv + kv head
    const int b = bh / p.hkv, kvh = bh % p.hkv;
    const int split = blockIdx.y;
    const int seq_len = p.seq_lens ? min(max(p.seq_lens[b], 0), p.s_max) : p.seq_len;
    const int n_chunks = (seq_len + CHUNK - 1) / CHUNK;
    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(n_chunks, c_begin + p.chunks_per_split);

    float scale_log2 = p.scale_log2;
    if (p.sq) scale_log2 *= __ldg(p.sq);
    if (p.sk) scale_log2 *= __ldg(p.sk);

    // Q fragments (A operand, 16 x D): rows g and g + 8 are query heads kvh*group + row of sequence b.
    // The contraction order over d is free, so the MMA's k index is fed a permutation of d that makes every lane's
    // share of a key row contiguous: lane t supplies d = (D/4)*t + 8*ks + {0..3} as k = 4t + {0..3} and
    // d = (D/4)*t + 8*ks + 4 + {0..3} as k = 16 + 4t + {0..3} of k-step ks, for Q (here) and K (below) alike; its K
    // fragments of all k-steps are then D/4 contiguous bytes (two 128-bit shared loads for D = 128).
    constexpr int KSTEPS = D / 32;
    uint32_t qa[KSTEPS][4];
    {
        const uint8_t* qb = p.q + ((size_t)b * p.hq + (size_t)kvh * p.group) * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int row = g + 8 * r;
                const bool live = row < p.group;
                qa[ks][r] = live ? *reinterpret_cast<const uint32_t*>(qb + (size_t)row * D + (D / 4) * t + 8 * ks) : 0u;
                qa[ks][2 + r] = live ? *reinterpret_cast<const uint32_t*>(qb + (size_t)row * D + (D / 4) * t + 8 * ks + 4) : 0u;
            }
        }
    }

    // online-softmax state of this warp for rows g and g + 8
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float oacc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; n++) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;

    // Each warp loads, converts and consumes its own 16 keys of every chunk (16 * D contiguous bytes of K and of V:
    // PER_THREAD 16-byte pieces per lane), so the loop needs only warp-level synchronisation and the four warps of a
    // CTA drift apart freely: their load latencies and MMA dependency stalls overlap instead of adding up.
    // The loop is issue-bound, so everything lane-constant is hoisted: 32-bit shared addresses, byte offsets of the
    // lane's pieces and fragments; only the last chunk of a sequence is masked.
    constexpr int PER_THREAD = 16 * D / 16 / 32;   // 4 (D = 128) or 2 (D = 64)
    constexpr int PARTS = D / 16;                   // 16-byte pieces per key row
    const uint32_t sm = smem_addr(smem);
    // piece i of this lane: key (16w + (32i + lane) / PARTS), part ((32i + lane) % PARTS); consecutive i are 32 pieces apart
    const int key_l = 16 * warp + lane / PARTS, part_l = lane % PARTS;
    const uint32_t k_dst = sm + key_l * S::K_STRIDE + part_l * 16;                      // + st * K_BYTES + i * (32 / PARTS) * K_STRIDE
    const uint32_t vraw = sm + S::OFF_VRAW + (key_l * PARTS + part_l) * 16;              // + st * VRAW_BYTES + i * 512
    const uint32_t k_frag = sm + (16 * warp + g) * S::K_STRIDE + (D / 4) * t;            // + st * K_BYTES + nt * 8 * K_STRIDE: D/4 bytes = all k-steps
    // ldmatrix.x4: lanes 0-15 address the 16 key rows at d-tile n, lanes 16-31 the same rows at d-tile n + 1
    const uint32_t v_frag = sm + S::OFF_V + (16 * warp + (lane & 15)) * S::V_STRIDE + (lane >> 4) * 16;   // + n * 16
    const size_t lane_goff = (size_t)(key_l * PARTS + part_l) * 16;                      // byte offset of piece 0 inside a chunk
    const uint8_t* kg = p.k + (PAGED ? 0 : (size_t)bh * p.s_max * D) + lane_goff;
    const uint8_t* vg = p.v + (PAGED ? 0 : (size_t)bh * p.s_max * D) + lane_goff;
    // paged: chunks are issued in order, so the position inside the block table advances incrementally (no division
    // per chunk), and the entry of the next page is fetched when the last chunk of the current page is issued: its
    // latency is hidden behind one loop iteration
    const int* table = nullptr;      // entry of the page the next chunk to be issued lives in
    int page_next = 0, within = 0;   // that entry's value; index of that chunk inside its page
    size_t head_off = 0, page_stride = 0;
    if (PAGED) {
        const int pg = c_begin / p.chunks_per_page;
        within = c_begin - pg * p.chunks_per_page;
        table = p.block_table + (size_t)b * p.max_pages + pg;
        if (c_begin < c_end) page_next = __ldg(table);
        page_stride = (size_t)p.hkv * p.page_size * D;
        head_off = (size_t)kvh * p.page_size * D;
    }
    auto issue_chunk = [&](int c) {   // global -> ring stage (c - c_begin) % STAGES, one commit group per chunk
        const int st = (c - c_begin) % STAGES;
        size_t off = (size_t)c * CHUNK * D;
        // keys at or past seq_len are not read but zero-filled: past s_max they would belong to the next head, and
        // below it they hold whatever the cache held before (possibly NaN codes; P = 0 there, but 0 x NaN would
        // still poison O).  Only a sequence's last chunk has such keys.
        const bool whole = (c + 1) * CHUNK <= seq_len;
        bool none = false;
        if (PAGED) {
            const int page = page_next;
            none = page < 0 || page >= p.num_pages;   // a table entry outside the pool: nothing is read, the keys count as zeros
            // a chunk never crosses a page (page_size is a multiple of CHUNK)
            off = none ? 0 : (size_t)page * page_stride + head_off + (size_t)within * (CHUNK * D);
            if (++within == p.chunks_per_page) {
                within = 0;
                ++table;
                if (c + 1 < c_end) page_next = __ldg(table);
            }
        }
#pragma unroll
        for (int i = 0; i < PER_THREAD; i++) {
            const uint32_t nbytes = (!none && (whole || c * CHUNK + key_l + i * (32 / PARTS) < seq_len)) ? 16u : 0u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(k_dst + st * S::K_BYTES + i * (32 / PARTS) * S::K_STRIDE),
                         "l"(kg + off + i * 512), "r"(nbytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vraw + st * S::VRAW_BYTES + i * 512), "l"(vg + off + i * 512), "r"(nbytes)
                         : "memory");
        }
    };
    auto commit = [&]() { asm volatile("cp.async.commit_group;" ::: "memory"); };
    // V codes of the landed stage -> fp16 copy the P V fragments are read from
    auto convert_v = [&](int st) {
        // lane j of the 8 (4) lanes of a key row converts codes [8j, 8j+8) and [D/2 + 8j, D/2 + 8j + 8): each of its two
        // 16-byte stores then lands next to its neighbours' (bank-conflict free), unlike a 32-byte run per lane
#pragma unroll
        for (int i = 0; i < PER_THREAD; i++) {
            const uint32_t src = sm + S::OFF_VRAW + st * S::VRAW_BYTES + (key_l + i * (32 / PARTS)) * D + part_l * 8;
            const uint32_t dst = sm + S::OFF_V + (key_l + i * (32 / PARTS)) * S::V_STRIDE + part_l * 16;
#pragma unroll
            for (int hlf = 0; hlf < 2; hlf++) {
                uint32_t w[2], h[4];
                asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(src + hlf * (D / 2)));
#pragma unroll
                for (int k = 0; k < 2; k++)
                    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\tcvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
                        : "=r"(h[2 * k]), "=r"(h[2 * k + 1])
                        : "r"(w[k]));
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst + hlf * D), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
            }
        }
    };

    // prologue: STAGES - 1 chunks in flight (empty groups keep the group count uniform)
#pragma unroll
    for (int i = 0; i < STAGES - 1; i++) {
        if (c_begin + i < c_end) issue_chunk(c_begin + i);
        commit();
    }
    for (int c = c_begin; c < c_end; c++) {
        const int st = (c - c_begin) % STAGES;
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");   // chunk c has landed (this lane's pieces)
        __syncwarp();             // ... the whole warp's pieces; and every lane is done with the previous chunk's fragments
        convert_v(st);
        if (c + STAGES - 1 < c_end) issue_chunk(c + STAGES - 1);   // into the stage computed one iteration ago
        commit();
        __syncwarp();

        // ---- S = Q K^T for this warp's 16 keys: two n-tiles of 8 keys.
        // one accumulator per (n-tile, k-step): eight independent MMAs instead of two chains of four (the legacy
        // mma.sync path has a 63-clock dependent-issue latency here), summed afterwards
        float s[2][4];
        {
            float part[2][KSTEPS][4];
            const uint32_t kf = k_frag + st * S::K_BYTES;
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                // B fragments of every k-step: key = column g of the n-tile, this lane's D/4 contiguous bytes of its row
                uint32_t kw[D / 16];
#pragma unroll
                for (int v = 0; v < D / 64; v++)
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(kw[4 * v]), "=r"(kw[4 * v + 1]), "=r"(kw[4 * v + 2]), "=r"(kw[4 * v + 3])
                                 : "r"(kf + nt * 8 * S::K_STRIDE + 16 * v));
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) mma_e4m3_m16n8k32_zero(part[nt][ks], qa[ks], kw[2 * ks], kw[2 * ks + 1]);
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float acc = part[nt][0][e];
#pragma unroll
                    for (int ks = 1; ks < KSTEPS; ks++) acc += part[nt][ks][e];
                    s[nt][e] = acc * scale_log2;
                }
        }
        // scores: s[nt][0..1] = row g, keys 8nt + 2t, +1 ; s[nt][2..3] = row g + 8
        if ((c + 1) * CHUNK > seq_len) {   // only the last chunk of a sequence has keys past its end
            const int key0 = c * CHUNK + 16 * warp;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (key0 + 8 * nt + 2 * t + (e & 1) >= seq_len) s[nt][e] = -INFINITY;
        }
        float mx[2];
        mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            corr[r] = (m[r] == -INFINITY) ? 0.f : ex2f(m[r] - m_new);   // m_new = -inf only if m is too
            m[r] = m_new;
        }
        uint32_t pa[4];
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                pv[e] = (m[e >> 1] == -INFINITY) ? 0.f : ex2f(s[nt][e] - m[e >> 1]);
                psum[e >> 1] += pv[e];
            }
            // A fragment of the 16 x 16 P tile: a0 = (row g, keys 2t..), a1 = (row g+8, ...), a2/a3 = keys + 8
            pa[2 * nt] = pack_h2(pv[0], pv[1]);
            pa[2 * nt + 1] = pack_h2(pv[2], pv[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
            psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
            l[r] = l[r] * corr[r] + psum[r];
        }
        // ---- O = O * corr + P V over this warp's 16 keys (the running maxima rarely move once a few chunks are in)
        const bool rescale = !__all_sync(0xffffffffu, corr[0] == 1.0f && corr[1] == 1.0f);
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, v_frag + n * 16);
            if (rescale) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    oacc[n + h][0] *= corr[0];
                    oacc[n + h][1] *= corr[0];
                    oacc[n + h][2] *= corr[1];
                    oacc[n + h][3] *= corr[1];
                }
            }
            mma_f16_m16n8k16(oacc[n], pa, b0, b1);
            mma_f16_m16n8k16(oacc[n + 1], pa, b2, b3);
        }
    }

    // ---- merge the four warps' states (shared memory reused)
    __syncthreads();
    float* mo = reinterpret_cast<float*>(smem);            // [4][ROWS][D]
    float* mml = mo + 4 * ROWS * D;                        // [4][ROWS][2]
#pragma unroll
    for (int n = 0; n < D / 8; n++) {
        float* base = mo + ((size_t)warp * ROWS) * D + n * 8 + 2 * t;
        base[(size_t)g * D] = oacc[n][0];
        base[(size_t)g * D + 1] = oacc[n][1];
        base[(size_t)(g + 8) * D] = oacc[n][2];
        base[(size_t)(g + 8) * D + 1] = oacc[n][3];
    }
    if (t == 0) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mml[(warp * ROWS + g + 8 * r) * 2] = m[r];
            mml[(warp * ROWS + g + 8 * r) * 2 + 1] = l[r];
        }
    }
    __syncthreads();
    const float vds = p.sv ? p.v_descale * __ldg(p.sv) : p.v_descale;
    for (int idx = threadIdx.x; idx < ROWS * D; idx += THREADS) {
        const int row = idx / D, col = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, mml[(w * ROWS + row) * 2]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float mw = mml[(w * ROWS + row) * 2];
            const float f = (mw == -INFINITY) ? 0.f : ex2f(mw - M);
            L += mml[(w * ROWS + row) * 2 + 1] * f;
            O += mo[((size_t)w * ROWS + row) * D + col] * f;
        }
        if (p.splits > 1) {
            const size_t slot = ((size_t)bh * p.splits + split) * ROWS + row;
            p.ws_o[slot * D + col] = O;
            if (col == 0) {
                p.ws_ml[slot * 2] = M;
                p.ws_ml[slot * 2 + 1] = L;
            }
        } else if (row < p.group) {
            const size_t orow = (size_t)b * p.hq + (size_t)kvh * p.group + row;
            p.o[orow * D + col] = __float2half_rn(L > 0.f ? O * (vds / L) : 0.f);
            if (col == 0 && p.lse) p.lse[orow] = (L > 0.f) ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        }
    }
}

// merges the splits of one (sequence, kv head): grid = B*Hkv, threads over ROWS x D
template <int D>
__global__ void __launch_bounds__(THREADS) fa_decode_combine_kernel(const DecodeParams p) {
    const int bh = blockIdx.x;
    const int b = bh / p.hkv, kvh = bh % p.hkv;
    const float vds = p.sv ? p.v_descale * __ldg(p.sv) : p.v_descale;
    for (int idx = threadIdx.x; idx < p.group * D; idx += THREADS) {
        const int row = idx / D, col = idx % D;
        float M = -INFINITY;
        for (int s = 0; s < p.splits; s++) M = fmaxf(M, p.ws_ml[(((size_t)bh * p.splits + s) * ROWS + row) * 2]);
        float L = 0.f, O = 0.f;
        for (int s = 0; s < p.splits; s++) {
            const size_t slot = ((size_t)bh * p.splits + s) * ROWS + row;
            const float ms = p.ws_ml[slot * 2];
            const float f = (ms == -INFINITY) ? 0.f : ex2f(ms - M);
            L += p.ws_ml[slot * 2 + 1] * f;
            O += p.ws_o[slot * D + col] * f;
        }
        const size_t orow = (size_t)b * p.hq + (size_t)kvh * p.group + row;
        p.o[orow * D + col] = __float2half_rn(L > 0.f ? O * (vds / L) : 0.f);
        if (col == 0 && p.lse) p.lse[orow] = (L > 0.f) ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
    }
}

int num_sms_of_current_device() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

}  // namespace

namespace {
int decode_splits(int batch, int kv_heads, int span) {
    // Enough CTAs to fill the GPU once (CTAS_PER_SM fit an SM) and no more: all of them resident at the same time, equal
    // key ranges, so none waits for a second wave; with batch * kv_heads CTAs or more there is nothing to split.
    const int chunks = (span + CHUNK - 1) / CHUNK;
    const long long ctas = (long long)batch * kv_heads;
    const long long slots = (long long)CTAS_PER_SM * num_sms_of_current_device();
    long long splits = slots / ctas;
    if (splits > chunks) splits = chunks;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    return (int)splits;
}
}  // namespace

size_t decode_workspace_bytes(int batch, int kv_heads, int head_dim, int span) {
    const int splits = decode_splits(batch, kv_heads, span);
    if (splits <= 1) return 0;
    return (size_t)batch * kv_heads * splits * ROWS * (head_dim + 2) * sizeof(float);
}

cudaError_t launch_decode(const DecodeArgs& a) {
    DecodeParams p;
    p.q = static_cast<const uint8_t*>(a.q);
    p.k = static_cast<const uint8_t*>(a.k_cache);
    p.v = static_cast<const uint8_t*>(a.v_cache);
    p.o = static_cast<__half*>(a.o);
    p.lse = a.lse;
    p.seq_lens = a.seq_lens;
    p.batch = a.batch; p.hq = a.q_heads; p.hkv = a.kv_heads; p.group = a.q_heads / a.kv_heads;
    p.s_max = a.s_max; p.seq_len = a.seq_len;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.v_descale = a.v_descale;
    p.sq = a.scale_q_dev; p.sk = a.scale_k_dev; p.sv = a.scale_v_dev;
    const int span = decode_span(a);
    p.splits = decode_splits(a.batch, a.kv_heads, span);
    const int chunks = (span + CHUNK - 1) / CHUNK;
    p.chunks_per_split = (chunks + p.splits - 1) / p.splits;
    p.ws_o = static_cast<float*>(a.workspace);
    p.ws_ml = p.ws_o ? p.ws_o + (size_t)a.batch * a.kv_heads * p.splits * ROWS * a.hd : nullptr;
    if (p.splits > 1 && !a.workspace) return cudaErrorInvalidValue;
    p.block_table = a.block_table;
    p.page_size = a.page_size; p.max_pages = a.max_pages; p.num_pages = a.num_pages;
    p.chunks_per_page = a.block_table ? a.page_size / CHUNK : 1;
    const dim3 grid((unsigned)(a.batch * a.kv_heads), (unsigned)p.splits);
    auto run = [&](auto kernel, auto combine, int smem_bytes) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        kernel<<<grid, THREADS, smem_bytes, a.stream>>>(p);
        if (p.splits > 1) combine<<<grid.x, THREADS, 0, a.stream>>>(p);
        return cudaSuccess;
    };
    cudaError_t e;
    if (a.hd == 128)
        e = a.block_table ? run(fa_decode_kernel<128, true>, fa_decode_combine_kernel<128>, Smem<128>::BYTES)
                          : run(fa_decode_kernel<128, false>, fa_decode_combine_kernel<128>, Smem<128>::BYTES);
    else
        e = a.block_table ? run(fa_decode_kernel<64, true>, fa_decode_combine_kernel<64>, Smem<64>::BYTES)
                          : run(fa_decode_kernel<64, false>, fa_decode_combine_kernel<64>, Smem<64>::BYTES);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

}  // namespace fa_sm100
