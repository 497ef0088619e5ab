"""Compile the sm_100a shared libraries in-tree with nvcc.

The libraries carry the file names goml's loaders look for
(backend/cuda/arch.go:84-101 resolves ``libfp8gemm.so`` inside a ``libs``
directory; backend/cuda/fa_forward.go:76-98 looks for ``libfa_sm120.so``).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBS = os.path.join(HERE, "libs")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-cudart", "static",
]

# library file -> sources
TARGETS = {
    "libfp8gemm.so": ["fp8_gemm_sm100.cu", "fp8_gemm_mx_sm100.cu"],
    "libfa_sm120.so": ["fa_api.cu", "fa_fwd_sm100.cu", "fa_decode_sm100.cu", "fa_dispatch.cpp"],
    "libfp8quant.so": ["fp8_quantize_sm100.cu"],
    "libfp8block.so": ["fp8_block_glue_sm100.cu"],
}


def _stale(out: str, srcs: list[str]) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = list(srcs)
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h")):
            deps.append(os.path.join(CSRC, f))
    inc = os.path.join(HERE, "..", "include")
    for f in os.listdir(inc):
        deps.append(os.path.join(inc, f))
    return any(os.path.getmtime(d) > t for d in deps)


def build_all(force: bool = False, verbose: bool = False, only: list[str] | None = None) -> list[str]:
    os.makedirs(LIBS, exist_ok=True)
    built = []
    for lib, srcs in TARGETS.items():
        if only and lib not in only:
            continue
        paths = [os.path.join(CSRC, s) for s in srcs]
        if not all(os.path.exists(p) for p in paths):
            continue
        out = os.path.join(LIBS, lib)
        if not force and not _stale(out, paths):
            continue
        cmd = ["nvcc", *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", out, *paths]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {lib}:\n{r.stdout}\n{r.stderr}")
        built.append(out)
    # north_star names the attention library by the glob libflash_attention*.so: the FP8 forward is reachable under
    # that family name too
    alias = os.path.join(LIBS, "libflash_attention_fp8.so")
    if os.path.exists(os.path.join(LIBS, "libfa_sm120.so")) and not os.path.lexists(alias):
        os.symlink("libfa_sm120.so", alias)
    return built


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print("built", p)
