#!/usr/bin/env bash
# build_cuda.sh — builds the B200 (sm_100a) libraries of the FP8 attention / FP8 GEMM path with plain nvcc.
#
# The counterpart of goml's scripts/build_cuda.sh for these four libraries.  It is meant to be dropped into a goml
# checkout (as scripts/build_cuda_b200.sh, with CSRC / INCLUDE / LIBS_DIR pointing at wherever the sources were
# placed) or run from this repository as it stands:
#
#     bash goml_b200/build_cuda.sh [all|fp8gemm|fa|quant|block]
#
# Environment (the names goml's Makefile already exports, scripts/build_cuda.sh:87 and Makefile:22-32):
#   GOML_TARGET_ONLY     when set, REPLACES the default gencode list.  goml's own script never reads this variable, so
#                        `make cuda-blackwell` / `make cuda-ampere` there do not restrict anything; this script does.
#                        The kernels use tcgen05 / TMEM instructions that exist only on the architecture-specific
#                        target sm_100a, so a value that names no compute_100a target is refused.
#   GOML_GENCODE_EXTRA   appended to the gencode list (e.g. an extra "a" target of a later part).
#   LIBS_DIR             output directory (default: goml_b200/libs beside this script; goml's loader looks in ./libs).
#   NVCC                 compiler (default: nvcc).
set -euo pipefail

HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
CSRC="${CSRC:-$HERE/csrc}"
LIBS_DIR="${LIBS_DIR:-$HERE/libs}"
NVCC="${NVCC:-nvcc}"

command -v "$NVCC" >/dev/null || { echo "ERROR: $NVCC not found" >&2; exit 1; }
CUDA_VERSION="$("$NVCC" --version | sed -n 's/.*release \([0-9]*\.[0-9]*\).*/\1/p')"
CUDA_MAJOR="${CUDA_VERSION%%.*}"; CUDA_MINOR="${CUDA_VERSION##*.}"
if [ "$CUDA_MAJOR" -lt 12 ] || { [ "$CUDA_MAJOR" -eq 12 ] && [ "$CUDA_MINOR" -lt 8 ]; }; then
    echo "ERROR: CUDA $CUDA_VERSION cannot target sm_100a (needs 12.8 or newer)" >&2; exit 1
fi

DEFAULT_GENCODE="-gencode arch=compute_100a,code=sm_100a"
GENCODE="${GOML_TARGET_ONLY:-$DEFAULT_GENCODE} ${GOML_GENCODE_EXTRA:-}"
case "$GENCODE" in
    *compute_100a*) ;;
    *) echo "ERROR: GOML_TARGET_ONLY='${GOML_TARGET_ONLY:-}' names no compute_100a target; these libraries are sm_100a-only" >&2; exit 2 ;;
esac

# -cudart static and hidden visibility: the libraries link nothing but the CUDA runtime and export only their C ABI,
# like the reference's (libs/fa_sm120/Makefile:12-14)
FLAGS="-O3 -std=c++17 -lineinfo --shared -Xcompiler -fPIC,-fvisibility=hidden -cudart static $GENCODE"

mkdir -p "$LIBS_DIR"
echo "=== goml FP8 path for B200 ===  nvcc $CUDA_VERSION   gencode:$GENCODE"
build() {   # output, sources...
    local out="$LIBS_DIR/$1"; shift
    local srcs=(); for s in "$@"; do srcs+=("$CSRC/$s"); done
    echo "  --> $out"
    "$NVCC" $FLAGS -o "$out" "${srcs[@]}"
}

TARGET="${1:-all}"
case "$TARGET" in all|fp8gemm) build libfp8gemm.so fp8_gemm_sm100.cu fp8_gemm_mx_sm100.cu ;; esac
case "$TARGET" in all|fa)      build libfa_sm120.so fa_api.cu fa_fwd_sm100.cu fa_decode_sm100.cu fa_dispatch.cpp
                               ln -sf libfa_sm120.so "$LIBS_DIR/libflash_attention_fp8.so" ;; esac   # reachable under the libflash_attention*.so family name too
case "$TARGET" in all|quant)   build libfp8quant.so fp8_quantize_sm100.cu ;; esac
case "$TARGET" in all|block)   build libfp8block.so fp8_block_glue_sm100.cu ;; esac
case "$TARGET" in all|fp8gemm|fa|quant|block) ;; *) echo "unknown target '$TARGET'" >&2; exit 2 ;; esac
echo "done."
