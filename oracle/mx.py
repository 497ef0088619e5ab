"""CPU restatement (numpy) of the block-scaled FP8 ("MXFP8") path.  TEST INFRASTRUCTURE ONLY.

The reference has no implementation of this path — only its roadmap entry (docs/FP8_FA_ROADMAP.md:137-148:
`kind::mxf8f6f4.block_scale.scale_vec::1X`, ue8m0 scale per 32 elements) — so this restates the published format
(OCP Microscaling Formats v1.0: shared scale 2^(floor(log2(amax)) - emax_elem) with emax_elem = 8 for e4m3, elements
rounded to nearest even and saturated) and parity is against this restatement only: PARITY UNPINNED.
"""
import numpy as np

import oracle as O

BLOCK = 32


def quantize_mx(x):
    """x [rows, K] float32 (K % 32 == 0) -> (codes uint8 [rows, K], scales uint8 [rows, K/32], ue8m0 = exponent + 127)."""
    x = np.ascontiguousarray(x, np.float32)
    rows, K = x.shape
    blocks = x.reshape(rows, K // BLOCK, BLOCK)
    amax = np.nanmax(np.abs(np.where(np.isnan(blocks), 0.0, blocks)), axis=-1)      # NaN never wins
    _, e = np.frexp(amax)                                 # amax = m * 2^e, m in [0.5, 1): floor(log2 amax) = e - 1
    se = np.where(amax > 0, e - 1 - 8, 0)
    se = np.where(np.isinf(amax), 127, se)
    se = np.clip(se, -127, 127).astype(np.int32)
    scaled = np.ldexp(blocks, -se[..., None]).astype(np.float32)
    codes = O.e4m3_encode(np.clip(scaled, -448.0, 448.0).reshape(rows, K))
    return codes, (se + 127).astype(np.uint8)


def dequantize_mx(codes, scales):
    """codes [rows, K], scales [rows, K/32] -> float64 values."""
    rows, K = codes.shape
    v = O.e4m3_decode(codes).astype(np.float64).reshape(rows, K // BLOCK, BLOCK)
    return np.ldexp(v, scales.astype(np.int32)[..., None] - 127).reshape(rows, K)


def gemm_mx_f64(a, sa, b, sb, alpha=1.0):
    """C = alpha * dequant(A) . dequant(B)^T in fp64 (the per-block scales are powers of two, so this equals
    sum over blocks of 2^(ea + eb) * (A_kb . B_kb))."""
    return alpha * (dequantize_mx(a, sa) @ dequantize_mx(b, sb).T)


def tile_scales(scales, K):
    """[rows, K/32] -> the byte order the kernel copies (include/fp8_gemm.h: fp8_gemm_mx): per 128-row tile and 128-element
    slab a 512-byte chunk, byte ((row % 32) * 16 + ((row % 128) / 32) * 4 + kb % 4); padding rows get scale 1 (0x7f)."""
    rows, kblocks = scales.shape
    assert K % 128 == 0 and kblocks == K // BLOCK
    rt, ks = (rows + 127) // 128, K // 128
    padded = np.full((rt * 128, kblocks), 0x7F, np.uint8)
    padded[:rows] = scales
    t = padded.reshape(rt, 4, 32, ks, 4)                   # [row tile, c = (row % 128) / 32, l = row % 32, slab, kb % 4]
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(-1)   # [row tile, slab, l, c, kb]
