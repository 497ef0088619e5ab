/*
 * oracle.c — CPU restatement of goml's FP8 attention-forward / FP8 GEMM / FP8
 * quantiser arithmetic.  TEST INFRASTRUCTURE ONLY: this file is the checker
 * the CUDA kernels are compared against and the timed CPU baseline.  Nothing
 * on the product path may call it.
 *
 * Every function cites the reference file:line whose arithmetic it follows
 * (paths are relative to the goml source tree).
 *
 * Parity pinning:
 *   - e4m3 decode, the harness attention reference and the harness GEMM
 *     reference are pinned against the reference's own CPU code (compiled from
 *     the reference tree into oracle/_ref by oracle/Makefile) and against the
 *     reference's known-answer tests (closed-form LSE, harness srand(42) grids).
 *   - e4m3 ENCODE (quantisation codes): no reference test pins codes
 *     ("parity unpinned" in the reference); the definition used here is the
 *     hardware one, round-to-nearest-even with saturation to +-448 and NaN ->
 *     0x7F (what __nv_fp8_e4m3(float) / cvt.rn.satfinite.e4m3x2 produce, which
 *     is what libs1/fp8_quantize_v2.cu:108-109 calls).  It is cross-checked
 *     against torch.float8_e4m3fn in the tests.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC -o liboracle.so oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ e4m3 */

/* Decode one e4m3 ("fn": no inf, NaN = S.1111.111) byte.
 * Follows backend/cuda/fa_contract_test.go:26-40 (e4m3Decode) and
 * libs/flash_attention_v121r_diet_hd128_fp8_forward.cu:697-703. */
ORACLE_API float oracle_e4m3_decode(uint8_t v)
{
    int s = (v >> 7) & 1, e = (v >> 3) & 0xF, m = v & 7;
    if (e == 0xF && m == 7) return NAN;
    float r = (e == 0) ? ldexpf((float)m, -9) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return s ? -r : r;
}

/* Encode fp32 -> e4m3, round-to-nearest-even, saturate-to-finite, subnormals
 * kept, NaN -> 0x7F.  This is the conversion libs1/fp8_quantize_v2.cu:108-109
 * performs through __nv_fp8_e4m3(float). */
ORACLE_API uint8_t oracle_e4m3_encode(float f)
{
    if (f != f) return 0x7F;
    uint8_t sign = signbit(f) ? 0x80 : 0x00;
    float a = fabsf(f);
    if (a >= 448.0f) return sign | 0x7E;            /* satfinite */
    if (a < 0.015625f) {                            /* below min normal 2^-6 */
        int q = (int)rintf(a * 512.0f);             /* units of 2^-9, RNE */
        return sign | (uint8_t)q;                   /* q == 8 is 0x08 = 2^-6 */
    }
    int e2;
    float fr = frexpf(a, &e2);                      /* a = fr * 2^e2, fr in [0.5,1) */
    int E = e2 - 1;                                 /* a = (2*fr) * 2^E */
    int q = (int)rintf(fr * 16.0f);                 /* mantissa in 1/8 steps, 8..16, RNE */
    if (q == 16) { q = 8; E += 1; }
    int code = ((E + 7) << 3) | (q - 8);
    if (code > 0x7E) code = 0x7E;
    return sign | (uint8_t)code;
}

ORACLE_API void oracle_e4m3_decode_n(const uint8_t *in, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = oracle_e4m3_decode(in[i]);
}

ORACLE_API void oracle_e4m3_encode_n(const float *in, uint8_t *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = oracle_e4m3_encode(in[i]);
}

/* ------------------------------------------------------------- quantiser */

/* Per-tensor quantiser.  Operation order follows
 * libs1/fp8_quantize_v2.cu:89-97 (scale) and :100-109 (x*inv, clamp, RN):
 *   amax  = max |x|
 *   scale = amax > 1e-12 ? amax / DIV : 1      (fp32 division)
 *   inv   = 1 / scale                           (fp32 division)
 *   q     = e4m3_rn(clamp(x * inv, -448, 448))
 * DIV = 448 is the reference quantiser (convention 0); DIV = 1 is the FA
 * magnitude contract "scale = amax" of libs/fa_sm120/include/fa_sm120.h:15-17
 * (convention 1: decoded magnitudes <= 1).  The reference reads fp16 input;
 * the inputs here are fp32 (internal/abjexam/battle_a_llm.go:463-494
 * quantises F32 activations). */
ORACLE_API void oracle_quantize_f32(const float *x, uint8_t *q, float *scale_out,
                                    float *amax_out, size_t n, int convention)
{
    float amax = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float a = fabsf(x[i]);
        if (a > amax) amax = a;                      /* NaN never wins, as fmaxf on device */
    }
    float div = (convention == 1) ? 1.0f : 448.0f;
    float scale = (amax > 1e-12f) ? (amax / div) : 1.0f;
    float inv = 1.0f / scale;
    for (size_t i = 0; i < n; i++) {
        float v = x[i] * inv;
        v = fminf(fmaxf(v, -448.0f), 448.0f);
        q[i] = oracle_e4m3_encode(v);
    }
    if (scale_out) *scale_out = scale;
    if (amax_out) *amax_out = amax;
}

/* -------------------------------------------------------------- attention */

/* FP64 attention forward on e4m3 codes.
 *   q,k,v  : [bh, sl, hd] codes;  scale = softmax_scale * scaleQ * scaleK
 *   o      : [bh, sl, hd] double, multiplied by v_descale
 *   lse    : [bh, sl] double natural-log LSE (may be NULL)
 * Arithmetic follows internal/f64ref/attention.go:42-88 (scores*scale, -inf
 * causal mask, P@V) and :160-191 (max-subtracted softmax; an all-masked row
 * yields zeros), on inputs decoded as backend/cuda/fa_contract_test.go:26-40.
 * LSE as defined at libs/fa_sm120/include/fa_sm120.h:100-102.
 * Mask: causal keeps keys j <= i; window > 0 additionally keeps only
 * j >= i - window + 1 (fa_sm120.h:76; harness reference
 * libs/flash_attention_v121r_diet_hd128_fp8_forward.cu:721-724).  With
 * causal = 0 and window > 0 the harness meaning is used: keys
 * [max(0, i-window+1), sl). */
ORACLE_API void oracle_attention_f64(const uint8_t *q, const uint8_t *k, const uint8_t *v,
                                     double *o, double *lse,
                                     int bh, int sl, int hd, int causal, int window,
                                     double scale, double v_descale)
{
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_decode((uint8_t)i);
    size_t hs = (size_t)sl * hd;
#pragma omp parallel
    {
        double *p = (double *)malloc(sizeof(double) * (size_t)sl);
        double *acc = (double *)malloc(sizeof(double) * (size_t)hd);
        float *kf = (float *)malloc(sizeof(float) * hs);
        float *vf = (float *)malloc(sizeof(float) * hs);
        for (int h = 0; h < bh; h++) {
            const uint8_t *Qh = q + h * hs, *Kh = k + h * hs, *Vh = v + h * hs;
            for (size_t i = 0; i < hs; i++) { kf[i] = lut[Kh[i]]; vf[i] = lut[Vh[i]]; }
#pragma omp for schedule(dynamic, 8)
            for (int i = 0; i < sl; i++) {
                int j1 = causal ? (i + 1) : sl;
                int j0 = (window > 0 && i + 1 > window) ? (i - window + 1) : 0;
                double qrow[256];
                for (int d = 0; d < hd; d++) qrow[d] = lut[Qh[(size_t)i * hd + d]];
                double mx = -INFINITY;
                for (int j = j0; j < j1; j++) {
                    const float *kr = kf + (size_t)j * hd;
                    double s = 0.0;
                    for (int d = 0; d < hd; d++) s += qrow[d] * (double)kr[d];
                    s *= scale;
                    p[j] = s;
                    if (s > mx) mx = s;
                }
                double *orow = o + h * hs + (size_t)i * hd;
                if (j1 <= j0 || isinf(mx)) {
                    for (int d = 0; d < hd; d++) orow[d] = 0.0;
                    if (lse) lse[(size_t)h * sl + i] = -INFINITY;
                    continue;
                }
                double sum = 0.0;
                for (int j = j0; j < j1; j++) { p[j] = exp(p[j] - mx); sum += p[j]; }
                for (int d = 0; d < hd; d++) acc[d] = 0.0;
                for (int j = j0; j < j1; j++) {
                    const float *vr = vf + (size_t)j * hd;
                    double pj = p[j];
                    for (int d = 0; d < hd; d++) acc[d] += pj * (double)vr[d];
                }
                double inv = v_descale / sum;
                for (int d = 0; d < hd; d++) orow[d] = acc[d] * inv;
                if (lse) lse[(size_t)h * sl + i] = mx + log(sum);
            }
        }
        free(p); free(acc); free(kf); free(vf);
    }
}

/* FP32 attention forward, the arithmetic of the reference's CPU paths:
 * backend/cpu/cpu.go:394-461 (float dot, *scale, softmax with float max and
 * float sum, P normalised before P@V) which is also what the kernel harness
 * reference libs/flash_attention_v121r_diet_hd128_fp8_forward.cu:709-752
 * (cpu_attention_fp8) does on decoded codes; the window rule is the
 * harness's (:721-724).  scale is passed in (both references use 1/sqrt(hd)).
 * Single-threaded per head exactly like the reference loops; heads are spread
 * over OpenMP threads only when parallel != 0. */
ORACLE_API void oracle_attention_f32(const uint8_t *q, const uint8_t *k, const uint8_t *v,
                                     float *o, int bh, int sl, int hd, int causal, int window,
                                     float scale, int parallel)
{
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_decode((uint8_t)i);
    size_t hs = (size_t)sl * hd;
#pragma omp parallel for schedule(dynamic, 1) if (parallel)
    for (int h = 0; h < bh; h++) {
        const uint8_t *Qh = q + h * hs, *Kh = k + h * hs, *Vh = v + h * hs;
        float *Oh = o + h * hs;
        float *P = (float *)malloc(sizeof(float) * (size_t)sl);
        for (int i = 0; i < sl; i++) {
            int j1 = causal ? (i + 1) : sl;
            int j0 = (window > 0 && i + 1 > window) ? (i - window + 1) : 0;
            float rmax = -1e30f;
            for (int j = j0; j < j1; j++) {
                float s = 0;
                for (int d = 0; d < hd; d++)
                    s += lut[Qh[(size_t)i * hd + d]] * lut[Kh[(size_t)j * hd + d]];
                P[j] = s * scale;
                if (P[j] > rmax) rmax = P[j];
            }
            float rsum = 0;
            for (int j = j0; j < j1; j++) { P[j] = expf(P[j] - rmax); rsum += P[j]; }
            for (int j = j0; j < j1; j++) P[j] /= rsum;
            for (int d = 0; d < hd; d++) {
                float acc = 0;
                for (int j = j0; j < j1; j++) acc += P[j] * lut[Vh[(size_t)j * hd + d]];
                Oh[(size_t)i * hd + d] = acc;
            }
        }
        free(P);
    }
}

/* ------------------------------------------------------------------- GEMM */

/* C[M,N] = alpha * sum_k A[m,k] * B[n,k] on e4m3 codes ("TN": both operands
 * K-contiguous), FP64 accumulation.  Follows internal/f64ref/linear.go:45-79
 * (y = x . W^T, W [out,in]) and internal/abjexam/battle_a_llm_f64ref.go:169-179
 * (matF64_ABT); operand layout as libs/fp8_gemm.cu:315-340. */
ORACLE_API void oracle_gemm_f64(const uint8_t *A, const uint8_t *B, double *C,
                                int M, int N, int K, double alpha)
{
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_decode((uint8_t)i);
    float *Af = (float *)malloc(sizeof(float) * (size_t)M * K);
    float *Bf = (float *)malloc(sizeof(float) * (size_t)N * K);
    for (size_t i = 0; i < (size_t)M * K; i++) Af[i] = lut[A[i]];
    for (size_t i = 0; i < (size_t)N * K; i++) Bf[i] = lut[B[i]];
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        const float *a = Af + (size_t)m * K;
        for (int n = 0; n < N; n++) {
            const float *b = Bf + (size_t)n * K;
            double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
            int kk = 0;
            for (; kk + 3 < K; kk += 4) {
                s0 += (double)a[kk] * b[kk];
                s1 += (double)a[kk + 1] * b[kk + 1];
                s2 += (double)a[kk + 2] * b[kk + 2];
                s3 += (double)a[kk + 3] * b[kk + 3];
            }
            for (; kk < K; kk++) s0 += (double)a[kk] * b[kk];
            C[(size_t)m * N + n] = alpha * ((s0 + s1) + (s2 + s3));
        }
    }
    free(Af); free(Bf);
}

/* FP32 GEMM exactly as the reference's own CPU check computes it:
 * libs/fp8_gemm_bench.cu:96-103 (float sum over k of decoded A[m,k]*B[n,k],
 * in k order, no scaling).  Rows are spread over OpenMP threads only when
 * parallel != 0 (each row's arithmetic is unchanged). */
ORACLE_API void oracle_gemm_f32(const uint8_t *A, const uint8_t *B, float *C,
                                int M, int N, int K, int parallel)
{
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_decode((uint8_t)i);
#pragma omp parallel for schedule(static) if (parallel)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float sum = 0;
            for (int kk = 0; kk < K; kk++)
                sum += lut[A[(size_t)m * K + kk]] * lut[B[(size_t)n * K + kk]];
            C[(size_t)m * N + n] = sum;
        }
}

/* ---------------------------------------------------------- harness data */

/* The reference self-check inputs: srand(42) then, per element i, Q,K,V drawn
 * in that interleaved order as ((rand()%16)-8)*0.125
 * (libs/flash_attention_v121r_diet_hd128_fp8_forward.cu:980-985).  All values
 * are exactly representable in e4m3, so any correct encoder gives the same
 * bytes.  glibc rand() makes this reproducible wherever glibc is. */
ORACLE_API void oracle_harness_attention_inputs(uint8_t *q, uint8_t *k, uint8_t *v, size_t n)
{
    srand(42);
    for (size_t i = 0; i < n; i++) {
        q[i] = oracle_e4m3_encode(((float)(rand() % 16) - 8.0f) * 0.125f);
        k[i] = oracle_e4m3_encode(((float)(rand() % 16) - 8.0f) * 0.125f);
        v[i] = oracle_e4m3_encode(((float)(rand() % 16) - 8.0f) * 0.125f);
    }
}

/* GEMM self-check inputs: srand(42), all of A then all of B as
 * ((rand()%16)-8)*0.25 (libs/fp8_gemm_bench.cu:91-95). */
ORACLE_API void oracle_harness_gemm_inputs(uint8_t *a, size_t na, uint8_t *b, size_t nb)
{
    srand(42);
    for (size_t i = 0; i < na; i++) a[i] = oracle_e4m3_encode(((float)(rand() % 16) - 8.0f) * 0.25f);
    for (size_t i = 0; i < nb; i++) b[i] = oracle_e4m3_encode(((float)(rand() % 16) - 8.0f) * 0.25f);
}

ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Same arithmetic as oracle_attention_f64, restricted to query rows
 * [q_begin, q_end) of every head (outputs are [bh, q_end-q_begin, hd] and
 * [bh, q_end-q_begin]).  Used to check full-size problems on a sample of rows. */
ORACLE_API void oracle_attention_f64_rows(const uint8_t *q, const uint8_t *k, const uint8_t *v,
                                          double *o, double *lse,
                                          int bh, int sl, int hd, int causal, int window,
                                          double scale, double v_descale, int q_begin, int q_end)
{
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_decode((uint8_t)i);
    size_t hs = (size_t)sl * hd;
    int nq = q_end - q_begin;
#pragma omp parallel
    {
        double *p = (double *)malloc(sizeof(double) * (size_t)sl);
        double *acc = (double *)malloc(sizeof(double) * (size_t)hd);
#pragma omp for collapse(2) schedule(dynamic, 4)
        for (int h = 0; h < bh; h++) {
            for (int qi = 0; qi < nq; qi++) {
                const uint8_t *Qh = q + h * hs, *Kh = k + h * hs, *Vh = v + h * hs;
                int i = q_begin + qi;
                int j1 = causal ? (i + 1) : sl;
                int j0 = (window > 0 && i + 1 > window) ? (i - window + 1) : 0;
                double qrow[256];
                for (int d = 0; d < hd; d++) qrow[d] = lut[Qh[(size_t)i * hd + d]];
                double mx = -INFINITY;
                for (int j = j0; j < j1; j++) {
                    const uint8_t *kr = Kh + (size_t)j * hd;
                    double s = 0.0;
                    for (int d = 0; d < hd; d++) s += qrow[d] * (double)lut[kr[d]];
                    s *= scale;
                    p[j] = s;
                    if (s > mx) mx = s;
                }
                double *orow = o + ((size_t)h * nq + qi) * hd;
                if (j1 <= j0 || isinf(mx)) {
                    for (int d = 0; d < hd; d++) orow[d] = 0.0;
                    if (lse) lse[(size_t)h * nq + qi] = -INFINITY;
                    continue;
                }
                double sum = 0.0;
                for (int j = j0; j < j1; j++) { p[j] = exp(p[j] - mx); sum += p[j]; }
                for (int d = 0; d < hd; d++) acc[d] = 0.0;
                for (int j = j0; j < j1; j++) {
                    const uint8_t *vr = Vh + (size_t)j * hd;
                    double pj = p[j];
                    for (int d = 0; d < hd; d++) acc[d] += pj * (double)lut[vr[d]];
                }
                double inv = v_descale / sum;
                for (int d = 0; d < hd; d++) orow[d] = acc[d] * inv;
                if (lse) lse[(size_t)h * nq + qi] = mx + log(sum);
            }
        }
        free(p); free(acc);
    }
}
