/*
 * ref_wrap_gemm.cu — exposes the reference's own host-side e4m3 helpers of the
 * FP8 GEMM self-check (libs/fp8_gemm_bench.cu:34-71) through a C ABI by
 * #including that file where it lies, main() renamed.  The CPU triple loop of
 * that self-check (libs/fp8_gemm_bench.cu:96-103) is not a function there, so
 * ref_gemm_cpu_loop below drives the reference's e4m3_to_float in the same
 * loop order.  The same translation unit also carries the reference's
 * mma.sync GEMM kernel entry fp8_gemm (libs/fp8_gemm.cu:315-340), re-exported
 * as ref_fp8_gemm so that "the reference kernel rebuilt for this GPU" can be
 * timed beside the new one.  TEST INFRASTRUCTURE ONLY; output to oracle/_ref/.
 */
#define main ref_gemm_bench_main
#include REF_GEMM_BENCH_SRC
#undef main

extern "C" {
/* the bench program itself (self-check at 128^3..512^3, then its shape table: libs/fp8_gemm_bench.cu:73-214) */
__attribute__((visibility("default")))
int ref_gemm_bench(int argc, char **argv) { (void)argc; (void)argv; return ref_gemm_bench_main(); }
__attribute__((visibility("default")))
uint8_t ref_gemm_float_to_e4m3(float f) { return float_to_e4m3(f); }
__attribute__((visibility("default")))
float ref_gemm_e4m3_to_float(uint8_t v) { return e4m3_to_float(v); }
__attribute__((visibility("default")))
void ref_gemm_cpu_loop(const uint8_t *hA, const uint8_t *hB, float *ref, int M, int N, int K)
{
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float sum = 0;
            for (int k = 0; k < K; k++)
                sum += e4m3_to_float(hA[m * K + k]) * e4m3_to_float(hB[n * K + k]);
            ref[m * N + n] = sum;
        }
}
__attribute__((visibility("default")))
int ref_fp8_gemm(int M, int N, int K, const void *A, const void *B, void *C, int mode, void *stream)
{
    return fp8_gemm(M, N, K, A, B, C, mode, stream);
}
}
