"""Runs the reference's own self-checking bench program for one of its GPU kernels, rebuilt for this GPU.

TEST INFRASTRUCTURE ONLY (never imported by the product).  oracle/Makefile compiles the reference's
FA harness files (libs/flash_attention_v121r_diet_hd128_fp8_forward.cu, libs/flash_attention_v89_pinregs_fp8_forward.cu)
and its GEMM bench (libs/fp8_gemm_bench.cu + libs/fp8_gemm.cu) for sm_100a with main() renamed; this script calls that
renamed main() with the given arguments, so "the reference kernel on this GPU" can be checked and timed with the
reference's own code:

    python oracle/ref_gpu_harness.py fa128                     # its 8-case self-check, then its bench table
    python oracle/ref_gpu_harness.py fa128 --time 128 8192 0   # median of 20 launches at bh=128, sl=8192, no window
    python oracle/ref_gpu_harness.py fa64
    python oracle/ref_gpu_harness.py gemm

The program's output goes to this process's stdout; its return code becomes the exit code.
"""
import ctypes as C
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIBS = {"fa128": ("libref_fa_hd128.so", "ref_fa_harness"), "fa64": ("libref_fa_hd64.so", "ref_fa_harness"),
        "gemm": ("libref_gemm.so", "ref_gemm_bench")}


def main(argv):
    if len(argv) < 2 or argv[1] not in LIBS:
        sys.stderr.write(__doc__)
        return 2
    name, entry = LIBS[argv[1]]
    path = os.path.join(HERE, "_ref", name)
    if not os.path.exists(path):
        sys.stderr.write(f"{path} is not built (make -C oracle, with the reference tree present)\n")
        return 3
    fn = getattr(C.CDLL(path), entry)
    fn.restype = C.c_int
    args = [name.encode()] + [a.encode() for a in argv[2:]]
    arr = (C.c_char_p * (len(args) + 1))(*args, None)
    sys.stdout.flush()
    rc = fn(len(args), arr)
    C.CDLL(None).fflush(None)
    return rc


if __name__ == "__main__":
    sys.exit(main(sys.argv))
