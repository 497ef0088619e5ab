"""Generates the golden fixtures in this directory FROM THE REFERENCE'S OWN CPU
CODE (oracle/_ref, compiled from the reference tree by oracle/Makefile).

Run where the reference tree is available:  python tests/golden/make_golden.py
The fixtures let the oracle be pinned on machines that have no reference tree.

Contents of reference_golden.npz
  e4m3_decode_table   reference e4m3_to_float over all 256 codes
  enc_in / enc_out    reference float_to_e4m3 on its own test grid (multiples of
                      1/8 and 1/4: the only values the reference feeds it)
  attn_<name>_o       reference cpu_attention_fp8 on the srand(42) harness inputs
                      for the reference's self-check shapes (bh,sl,hd,causal,window)
  gemm_128_ref        reference GEMM float loop on the srand(42) 128^3 inputs
  *_sha               sha256 of the srand(42) input bytes (pins the generator)
"""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle as O  # noqa: E402

ATTN_SHAPES = {
    "s64": (1, 64, 128, 0, 0), "s128": (1, 128, 128, 0, 0), "s256": (1, 256, 128, 0, 0),
    "c256": (2, 256, 128, 1, 0), "w64": (1, 256, 128, 1, 64), "w100": (1, 256, 128, 1, 100),
    "w96": (1, 300, 128, 1, 96), "hd64": (1, 256, 64, 0, 0), "hd64c": (2, 128, 64, 1, 0),
}


def main():
    R = O.ref()
    assert R.available, "oracle/_ref not built (needs the reference tree): make -C oracle"
    out = {}
    out["e4m3_decode_table"] = np.array([R.fa128.ref_e4m3_to_float(c) for c in range(256)], np.float32)
    grid = np.concatenate([(np.arange(16) - 8) * 0.125, (np.arange(16) - 8) * 0.25]).astype(np.float32)
    out["enc_in"] = grid
    out["enc_out"] = np.array([R.fa128.ref_float_to_e4m3(float(x)) for x in grid], np.uint8)
    for name, (bh, sl, hd, ca, w) in ATTN_SHAPES.items():
        q, k, v = O.harness_attention_inputs(bh, sl, hd)
        out[f"attn_{name}_o"] = R.cpu_attention_fp8(q, k, v, ca, w)
        out[f"attn_{name}_sha"] = np.frombuffer(hashlib.sha256(q.tobytes() + k.tobytes() + v.tobytes()).digest(), np.uint8)
    a, b = O.harness_gemm_inputs(128, 128, 128)
    out["gemm_128_ref"] = R.gemm_cpu_loop(a, b)
    out["gemm_128_sha"] = np.frombuffer(hashlib.sha256(a.tobytes() + b.tobytes()).digest(), np.uint8)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
