/*
 * ref_wrap_fa.cu — exposes the reference's OWN host-side CPU functions for the
 * FP8 attention path through a C ABI, without copying them: the reference
 * translation unit is #included where it lies (REF_FA_SRC is set by
 * oracle/Makefile to libs/flash_attention_v121r_diet_hd128_fp8_forward.cu or
 * its hd64 twin libs/flash_attention_v89_pinregs_fp8_forward.cu) with its
 * main() renamed.  TEST INFRASTRUCTURE ONLY (validates oracle.c; timed as the
 * "reference" CPU baseline).  Output goes to oracle/_ref/ only.
 */
#define main ref_harness_main
#include REF_FA_SRC
#undef main

extern "C" {
/* the harness program itself (self-check, bench table, --time/--ncu/--loop modes: same file :757-1130) */
__attribute__((visibility("default")))
int ref_fa_harness(int argc, char **argv) { return ref_harness_main(argc, argv); }
/* cpu_attention_fp8: .../flash_attention_v121r_diet_hd128_fp8_forward.cu:709-752 */
__attribute__((visibility("default")))
void ref_cpu_attention_fp8(const uint8_t *Q, const uint8_t *K, const uint8_t *V, float *O,
                           int bh, int sl, int hd, int causal, int window)
{
    cpu_attention_fp8(Q, K, V, O, bh, sl, hd, causal, window);
}
/* float_to_e4m3 / e4m3_to_float: same file :676-703 */
__attribute__((visibility("default")))
uint8_t ref_float_to_e4m3(float f) { return float_to_e4m3(f); }
__attribute__((visibility("default")))
float ref_e4m3_to_float(uint8_t v) { return e4m3_to_float(v); }
}
