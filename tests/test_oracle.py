"""The oracle pinned against the reference: golden vectors made by the
reference's own CPU code (tests/golden), that code itself where it is compiled
(oracle/_ref), the reference's known-answer tests, and torch's e4m3 casts."""
import hashlib
import math

import numpy as np
import pytest
import torch

import oracle as O
from tests.golden.make_golden import ATTN_SHAPES


def test_e4m3_decode_table_matches_reference(golden):
    got = O.e4m3_decode(np.arange(256, dtype=np.uint8))
    ref = golden["e4m3_decode_table"]
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert np.array_equal(got[~np.isnan(got)], ref[~np.isnan(ref)])
    # anchors quoted by backend/cuda/fa_forward_test.go:17-21
    assert got[0x38] == 1.0 and got[0x40] == 2.0 and got[0x48] == 4.0 and got[0x7E] == 448.0


def test_e4m3_encode_matches_reference_on_its_grid(golden):
    # the reference's host encoder is only ever fed exactly representable values;
    # on those any correct encoder agrees with it
    assert np.array_equal(O.e4m3_encode(golden["enc_in"]), golden["enc_out"])


def test_e4m3_encode_is_rne_satfinite_vs_torch():
    rng = np.random.default_rng(1)
    xs = [rng.standard_normal(200_000).astype(np.float32) * s for s in (1e-3, 0.02, 1.0, 30.0, 300.0)]
    h = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    xs.append(h[np.isfinite(h)])
    x = np.clip(np.concatenate(xs), -448, 448)  # torch's cast does not saturate
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x), want)
    # saturation, NaN, signed zero, ties-to-even at a midpoint
    assert list(O.e4m3_encode(np.array([1e9, -1e9, 449.0, 463.9, np.inf], np.float32))) == [0x7E, 0xFE, 0x7E, 0x7E, 0x7E]
    assert O.e4m3_encode(np.array([np.nan], np.float32))[0] == 0x7F
    assert list(O.e4m3_encode(np.array([0.0, -0.0], np.float32))) == [0x00, 0x80]
    assert list(O.e4m3_encode(np.array([1.0625, 1.1875], np.float32))) == [0x38, 0x3A]  # ties go to even mantissa


def test_e4m3_roundtrip_all_codes():
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    assert np.array_equal(O.e4m3_encode(O.e4m3_decode(codes)), codes)


@pytest.mark.parametrize("convention,div", [(0, 448.0), (1, 1.0)])
def test_quantizer_definition(convention, div):
    x = O.seeded_normal("x", (3, 1000), config="quant")
    q, scale, amax = O.quantize_f32(x, convention)
    assert amax == np.abs(x).max()
    assert scale == np.float32(amax) / np.float32(div)
    inv = np.float32(1.0) / scale
    y = np.clip(x * inv, -448, 448)
    want = torch.from_numpy(y).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(q, want)
    # the largest element maps to +-448 (convention 0) or +-1 (convention 1)
    assert np.abs(O.e4m3_decode(q)).max() == (448.0 if convention == 0 else 1.0)


def test_quantizer_zero_tensor_uses_unit_scale():
    q, scale, amax = O.quantize_f32(np.zeros(33, np.float32))
    assert scale == 1.0 and amax == 0.0 and not q.any()


@pytest.mark.parametrize("name", sorted(ATTN_SHAPES))
def test_attention_matches_reference_cpu_code(golden, name):
    bh, sl, hd, ca, w = ATTN_SHAPES[name]
    q, k, v = O.harness_attention_inputs(bh, sl, hd)
    sha = hashlib.sha256(q.tobytes() + k.tobytes() + v.tobytes()).digest()
    assert sha == golden[f"attn_{name}_sha"].tobytes(), "srand(42) harness inputs differ"
    ref = golden[f"attn_{name}_o"]
    # the fp32 restatement is bit-exact with the reference's cpu_attention_fp8
    assert np.array_equal(O.attention_f32(q, k, v, ca, w), ref)
    # the fp64 restatement agrees to fp32 rounding
    o64, _ = O.attention_f64(q, k, v, ca, w)
    assert np.abs(o64 - ref).max() < 2e-6
    o64r, _ = O.attention_f64_rows(q, k, v, 3, min(sl, 40), ca, w)
    assert np.array_equal(o64r, o64[:, 3:min(sl, 40)])


def test_gemm_matches_reference_cpu_code(golden):
    a, b = O.harness_gemm_inputs(128, 128, 128)
    assert hashlib.sha256(a.tobytes() + b.tobytes()).digest() == golden["gemm_128_sha"].tobytes()
    ref = golden["gemm_128_ref"]
    assert np.array_equal(O.gemm_f32(a, b), ref)
    assert np.array_equal(O.gemm_f64(a, b), ref.astype(np.float64))  # sums of 1/16 multiples are exact
    assert np.allclose(O.gemm_f64(a, b, alpha=0.5), 0.5 * ref)


def test_live_reference_code_if_compiled():
    R = O.ref()
    if not R.available:
        pytest.skip("oracle/_ref not built on this machine (no reference tree)")
    rng = np.random.default_rng(7)
    for bh, sl, hd, ca, w in [(2, 96, 128, 0, 0), (1, 200, 64, 1, 0), (1, 160, 128, 1, 50)]:
        q = rng.integers(0, 0x78, (bh, sl, hd), dtype=np.uint8) | (rng.integers(0, 2, (bh, sl, hd), dtype=np.uint8) << 7)
        k = rng.integers(0, 0x50, (bh, sl, hd), dtype=np.uint8)
        v = rng.integers(0, 0x78, (bh, sl, hd), dtype=np.uint8)
        assert np.array_equal(O.attention_f32(q, k, v, ca, w), R.cpu_attention_fp8(q, k, v, ca, w))
    a = rng.integers(0, 0x78, (40, 64), dtype=np.uint8)
    b = rng.integers(0, 0x78, (24, 64), dtype=np.uint8)
    assert np.array_equal(O.gemm_f32(a, b), R.gemm_cpu_loop(a, b))


def test_lse_closed_forms():
    # backend/cuda/fa_forward_test.go:112-189: all ones -> L = sqrt(hd) + ln(sl), O = 1
    q = np.full((3, 280, 128), 0x38, np.uint8)
    o, l = O.attention_f64(q, q, q)
    assert np.allclose(l, math.sqrt(128) + math.log(280), rtol=1e-12) and np.allclose(o, 1.0)
    # backend/cuda/fa_forward_test.go:191-288: Q = 1,2,4 per head -> L = 2^i sqrt(hd) + ln(sl)
    qh = np.stack([np.full((280, 128), c, np.uint8) for c in (0x38, 0x40, 0x48)])
    _, l = O.attention_f64(qh, q, q)
    for i in range(3):
        assert np.allclose(l[i], 2 ** i * math.sqrt(128) + math.log(280), rtol=1e-12)


def test_attention_masks_and_empty_rows():
    q, k, v = O.harness_attention_inputs(1, 64, 64)
    o, l = O.attention_f64(q, k, v, causal=1, window=1)  # each query sees only itself
    assert np.allclose(o[0], O.e4m3_decode(v[0]).astype(np.float64))
    # causal=0 with a window: keys [i-w+1, sl) (the harness meaning)
    o2, _ = O.attention_f64(q, k, v, causal=0, window=64)
    o3, _ = O.attention_f64(q, k, v, causal=0, window=0)
    assert np.allclose(o2, o3)


def test_output_rounding_helpers():
    x = np.array([1.0, 1.00390625, 3.14159, -2.5e-3, 65504.0], np.float64)
    want = torch.tensor(x, dtype=torch.float32).to(torch.bfloat16).float().numpy()
    assert np.array_equal(O.round_bf16(x), want)
    assert np.array_equal(O.round_fp16(x), torch.tensor(x).to(torch.float16).numpy())
    a = O.seeded_normal("t", (4, 5), config="c")
    assert np.array_equal(a, O.seeded_normal("t", (4, 5), config="c"))
    assert not np.array_equal(a, O.seeded_normal("u", (4, 5), config="c"))


def test_mx_restatement_properties():
    # block-scaled format: scales are the OCP shared exponents, elements stay within e4m3 range, dequantisation error is
    # bounded by half an e4m3 step of the block's largest element, and the tiled scale order is a permutation
    import numpy as np
    from oracle import mx
    x = (O.seeded_normal("x", (130, 256), config="mxcpu") * np.exp2(np.arange(256) // 32 - 4)[None, :]).astype(np.float32)
    x[3, :32] = 0
    codes, scales = mx.quantize_mx(x)
    assert codes.shape == x.shape and scales.shape == (130, 8) and scales[3, 0] == 127
    amax = np.abs(x).reshape(130, 8, 32).max(-1)
    nz = amax > 0
    assert np.all(np.exp2(scales.astype(int) - 127 + 8)[nz] <= amax[nz]) and np.all(amax[nz] < np.exp2(scales.astype(int) - 127 + 9)[nz])
    back = mx.dequantize_mx(codes, scales)
    err = np.abs(back - x).reshape(130, 8, 32).max(-1)
    # scaled elements reach [256, 512): half an e4m3 step there is 16, and what lies above 448 saturates (error < 64)
    assert np.all(err <= np.exp2(scales.astype(float) - 127) * 64) and np.median(err / np.exp2(scales.astype(float) - 127)) <= 16
    tiled = mx.tile_scales(scales, 256)
    assert tiled.size == 2 * 2 * 512
    assert tiled[(0 * 2 + 1) * 512 + 5 * 16 + 2 * 4 + 3] == scales[2 * 32 + 5, 4 + 3]     # row 69, block 7
    assert tiled[(1 * 2 + 0) * 512 + 1 * 16 + 0 * 4 + 0] == scales[129, 0] and tiled[(1 * 2 + 0) * 512 + 9 * 16] == 0x7F   # padding rows
    a, sa = mx.quantize_mx(O.seeded_normal("a", (4, 64), config="mxcpu"))
    b, sb = mx.quantize_mx(O.seeded_normal("b", (3, 64), config="mxcpu"))
    want = sum(np.ldexp(O.e4m3_decode(a[:, 32 * k:32 * k + 32]).astype(np.float64) @ O.e4m3_decode(b[:, 32 * k:32 * k + 32]).astype(np.float64).T,
                        (sa[:, k].astype(int)[:, None] - 127) + (sb[:, k].astype(int)[None, :] - 127)) for k in range(2))
    assert np.allclose(mx.gemm_mx_f64(a, sa, b, sb), want, rtol=1e-13)
