"""FP8 GEMM parity on the GPU, through the C ABI, against the oracle.

Tolerances.  The reference's own gate (libs/fp8_gemm_bench.cu:120-129) is
|gpu-ref| <= max(1.0, 0.05|ref|).  The bar used here for seeded N(0,1) data:
max-abs error <= 2e-2 and mean relative error <= 1e-2, both measured on C
normalised by RMS(C_ref) — at 4096^3 the un-normalised products have RMS ~ 64
where one bf16 step is 0.25, so an absolute 2e-2 is below the output format's
resolution.  In addition the result must equal the oracle's fp64 result rounded
to the output type up to one unit in the last place (accumulation is fp32).
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests.gpu_util import dev_u8, run_gemm

pytestmark = pytest.mark.gpu


def check(got, ref64, bf16):
    rms = np.sqrt(np.mean(ref64 ** 2))
    maxabs, meanrel = O.error_stats(got / rms, ref64 / rms)
    assert maxabs <= 2e-2, maxabs
    assert meanrel <= 1e-2, meanrel
    # within one ulp of the correctly rounded result
    ulp = np.abs(ref64) * (2.0 ** -7 if bf16 else 2.0 ** -10) + 1e-3 * rms  # floor: fp32 accumulation noise near 0
    assert np.all(np.abs(got - ref64) <= ulp)


@pytest.mark.parametrize("entry", ["gemm", "original", "singlesync"])
@pytest.mark.parametrize("n", [128, 256, 512])
def test_reference_selfcheck_shapes(cuda, built_libs, golden, entry, n):
    # libs/fp8_gemm_bench.cu:81-141: srand(42) inputs, 128^3/256^3/512^3, fp16 out
    a, b = O.harness_gemm_inputs(n, n, n)
    got = run_gemm(a, b, bf16=False, entry=entry)
    ref = O.gemm_f32(a, b, parallel=True).astype(np.float64)
    if n == 128:
        assert np.array_equal(ref, golden["gemm_128_ref"].astype(np.float64))
    assert np.all(np.abs(got - ref) <= np.maximum(1.0, 0.05 * np.abs(ref)))       # the reference's gate
    assert np.array_equal(got, O.round_fp16(ref).astype(np.float64))             # and in fact exact


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (1024, 1024, 1024), (384, 640, 2048)])
@pytest.mark.parametrize("bf16", [True, False])
def test_seeded_normal_amax448(cuda, built_libs, M, N, K, bf16):
    # config: A, B ~ N(0,1) quantised per tensor with scale = amax/448; C = sa*sb * A.B^T
    a, sa, _ = O.quantize_f32(O.seeded_normal("A", (M, K), config=f"gemm{M}x{N}x{K}"))
    b, sb, _ = O.quantize_f32(O.seeded_normal("B", (N, K), config=f"gemm{M}x{N}x{K}"))
    alpha = float(sa) * float(sb)
    got = run_gemm(a, b, alpha=alpha, bf16=bf16)
    check(got, O.gemm_f64(a, b, alpha), bf16)


def test_device_scale_pointers(cuda, built_libs):
    a, sa, _ = O.quantize_f32(O.seeded_normal("A", (128, 256), config="ptr"))
    b, sb, _ = O.quantize_f32(O.seeded_normal("B", (256, 256), config="ptr"))
    s = torch.tensor([float(sa), float(sb)], dtype=torch.float32, device="cuda")
    got = run_gemm(a, b, alpha=1.0, scale_ptrs=(s.data_ptr(), s.data_ptr() + 4))
    check(got, O.gemm_f64(a, b, float(np.float32(sa) * np.float32(sb))), True)


@pytest.mark.parametrize("M,N,K", [(1, 8, 16), (16, 8192, 256), (129, 257, 160), (300, 520, 144), (127, 255, 4096),
                                    (130, 7, 48), (5, 1000, 16),
                                    # 150 / 190 tiles of 128x256 on 148 SMs: the last wave runs as half-width units
                                    (256, 19200, 160), (640, 9700, 144)])
def test_ragged_and_tiny_shapes(cuda, built_libs, M, N, K):
    rng = np.random.default_rng(M * 1000 + N)
    a = rng.integers(0, 0x7F, (M, K), dtype=np.uint8) | (rng.integers(0, 2, (M, K), dtype=np.uint8) << 7)
    b = rng.integers(0, 0x60, (N, K), dtype=np.uint8) | (rng.integers(0, 2, (N, K), dtype=np.uint8) << 7)
    alpha = 2.0 ** -10
    got = run_gemm(a, b, alpha=alpha, bf16=True)
    check(got, O.gemm_f64(a, b, alpha), True)


def test_output_outside_the_matrix_is_untouched(cuda, built_libs):
    from goml_b200 import fp8_gemm as G
    M, N, K = 100, 72, 64
    a, b = O.harness_gemm_inputs(M, N, K)
    ad, bd = dev_u8(a), dev_u8(b)
    buf = torch.full((M * N + 512,), 7.0, dtype=torch.float16, device="cuda")
    G.FP8GEMM(M, N, K, ad.data_ptr(), bd.data_ptr(), buf.data_ptr() + 512, 1, 0)   # C starts 256 elements in
    torch.cuda.synchronize()
    assert torch.all(buf[:256] == 7.0) and torch.all(buf[256 + M * N:] == 7.0)
    ref = O.round_fp16(O.gemm_f32(a, b)).astype(np.float64)
    assert np.array_equal(buf[256:256 + M * N].double().cpu().numpy().reshape(M, N), ref)


def test_fp32_accumulation_does_not_overflow_like_fp16(cuda, built_libs):
    # all codes 0x7E (448): 448*448*K overflows an fp16 accumulator; alpha brings the result into range
    K = 256
    a = np.full((128, K), 0x7E, np.uint8)
    b = np.full((256, K), 0x7E, np.uint8)
    got = run_gemm(a, b, alpha=2.0 ** -16, bf16=True)
    assert np.allclose(got, 448.0 * 448.0 * K * 2.0 ** -16, rtol=2 ** -8)


def test_config2_full_size_on_sampled_rows(cuda, built_libs):
    # M=N=K=4096, bf16 out scaled by sa*sb; oracle on 48 sampled rows (all columns)
    from goml_b200 import fp8_gemm as G
    n = 4096
    a, sa, _ = O.quantize_f32(O.seeded_normal("A", (n, n), config="C2"))
    b, sb, _ = O.quantize_f32(O.seeded_normal("B", (n, n), config="C2"))
    alpha = float(sa) * float(sb)
    ad, bd = dev_u8(a), dev_u8(b)
    c = torch.empty((n, n), dtype=torch.bfloat16, device="cuda")
    G.FP8GEMMScaled(n, n, n, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), alpha, 0, 0, G.OutBF16, 0)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    rows = np.unique(np.concatenate([[0, 127, 128, 4095], np.random.default_rng(0).integers(0, n, 44)]))
    got = c[torch.from_numpy(rows).cuda()].double().cpu().numpy()
    check(got, O.gemm_f64(a[rows], b, alpha), True)
    # size-independent property: C is linear in alpha (same bits scaled by a power of two)
    c2 = torch.empty_like(c)
    G.FP8GEMMScaled(n, n, n, ad.data_ptr(), bd.data_ptr(), c2.data_ptr(), alpha * 4.0, 0, 0, G.OutBF16, 0)
    torch.cuda.synchronize()
    assert torch.equal(c2, c * 4.0)
    # and rows of A map to rows of C: a row permutation of A permutes C
    perm = torch.randperm(n, device="cuda")
    c3 = torch.empty_like(c)
    G.FP8GEMMScaled(n, n, n, ad[perm].contiguous().data_ptr(), bd.data_ptr(), c3.data_ptr(), alpha, 0, 0, G.OutBF16, 0)
    torch.cuda.synchronize()
    assert torch.equal(c3, c[perm])


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (300, 520, 144), (129, 257, 160), (16, 8192, 256),
                                   (16, 4096, 4096), (48, 1024, 11008), (16, 512, 2064)])      # the last three run split over K
def test_accumulate_into_fp32(cuda, built_libs, M, N, K):
    # the residual-stream update in the epilogue: X += alpha * sa * sb * A.B^T, fp32 accumulators added un-rounded
    from goml_b200 import fp8_gemm as G
    cfg = f"acc{M}x{N}x{K}"
    a, sa, _ = O.quantize_f32(O.seeded_normal("A", (M, K), config=cfg))
    b, sb, _ = O.quantize_f32(O.seeded_normal("B", (N, K), config=cfg))
    x = O.seeded_normal("X", (M, N), config=cfg).astype(np.float32)
    ad, bd = dev_u8(a), dev_u8(b)
    xd = torch.from_numpy(x.copy()).cuda()
    scales = torch.tensor([float(sa), float(sb)], dtype=torch.float32, device="cuda")
    G.FP8GEMMAccumulateF32(M, N, K, ad.data_ptr(), bd.data_ptr(), xd.data_ptr(), 0.5, scales.data_ptr(), scales.data_ptr() + 4)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    prod = O.gemm_f64(a, b, 0.5 * float(np.float32(sa) * np.float32(sb)))
    ref = x.astype(np.float64) + prod
    got = xd.double().cpu().numpy()
    rms = float(np.sqrt(np.mean(prod ** 2)))
    assert np.abs(got - ref).max() <= 1e-5 * max(rms, 1.0) * np.sqrt(K), np.abs(got - ref).max()


@pytest.mark.parametrize("M,F,K", [(256, 1376, 512), (130, 704, 256), (64, 11008, 128), (300, 128, 144),
                                   (2048, 2440, 128), (520, 4096, 256)])     # wide tiles: H leaves through TMA stores, clipped at column F
def test_swiglu_epilogue(cuda, built_libs, M, F, K):
    # gate/up projections with silu(gate) * up in the epilogue: bf16 H, max|H| exact, and the quantiser pass that follows
    from goml_b200 import fp8_gemm as G, block_glue as BG
    cfg = f"swiglu{M}x{F}x{K}"
    a, sa, _ = O.quantize_f32(O.seeded_normal("A", (M, K), config=cfg))
    w, sw, _ = O.quantize_f32(O.seeded_normal("W", (2 * F, K), std=0.08, config=cfg))
    wi = G.interleave_gate_up(w, F)
    ad, wd = dev_u8(a), dev_u8(wi)
    h = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    scales = torch.tensor([float(sa), float(sw)], dtype=torch.float32, device="cuda")
    s2 = torch.full((2,), 5.0, dtype=torch.float32, device="cuda")
    G.FP8GEMMSwiGLU(M, F, K, ad.data_ptr(), wd.data_ptr(), h.data_ptr(), 1.0, scales.data_ptr(), scales.data_ptr() + 4, s2.data_ptr() + 4)
    q = torch.full((M, F), 0xAA, dtype=torch.uint8, device="cuda")
    BG.QuantizeBF16(h.data_ptr(), q.data_ptr(), s2.data_ptr(), s2.data_ptr() + 4, M * F)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    gu = O.gemm_f64(a, w, float(np.float32(sa) * np.float32(sw)))
    g, u = gu[:, :F], gu[:, F:]
    ref = g / (1.0 + np.exp(-g)) * u
    got = h.double().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.all(np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-6 * np.abs(ref).max())
    hv = h.float().cpu().numpy()
    assert s2[1].item() == np.abs(hv).max()                       # the epilogue's amax is the max of what it wrote
    codes, scale, amax = O.quantize_f32(np.ascontiguousarray(hv))
    assert s2[0].item() == scale and np.array_equal(q.cpu().numpy(), codes)   # quantiser pass bit-exact on those values


def _fp8out(a, b, alpha, sa, sb, sd, want_amax=True, guard=0):
    """Run fp8_gemm_fp8out on host codes a [M,K], b [N,K]; returns (codes [M,N] (+guard bytes), amax)."""
    from goml_b200 import fp8_gemm as G
    M, K = a.shape
    N = b.shape[0]
    ad, bd = dev_u8(a), dev_u8(b)
    d = torch.full((M * N + guard,), 0xAA, dtype=torch.uint8, device="cuda")
    s = torch.tensor([sa, sb, sd, 123.0], dtype=torch.float32, device="cuda")
    G.FP8GEMMFP8Out(M, N, K, ad.data_ptr(), bd.data_ptr(), d.data_ptr(), alpha, s.data_ptr(), s.data_ptr() + 4,
                    s.data_ptr() + 8, s.data_ptr() + 12 if want_amax else 0)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    return d.cpu().numpy(), float(s[3].item())


@pytest.mark.parametrize("M,N,K", [(256, 512, 512), (130, 272, 144), (129, 250, 160), (16, 8192, 256), (300, 24, 1024),
                                   (2048, 4880, 128), (520, 4096, 256)])     # wide tiles: D leaves through TMA stores, clipped at column N
def test_fp8out_exact_on_integer_data(cuda, built_libs, M, N, K):
    # small-integer operands: every partial sum is exact in fp32, so the e4m3 codes and amax must be bit-exact
    rng = np.random.default_rng(M * 7 + N)
    av = rng.integers(-3, 4, size=(M, K)).astype(np.float32)
    bv = rng.integers(-3, 4, size=(N, K)).astype(np.float32)
    a, b = O.e4m3_encode(av), O.e4m3_encode(bv)
    assert np.array_equal(O.e4m3_decode(a), av)
    alpha, sa, sb, sd = np.float32(0.25), np.float32(0.5), np.float32(1.5), np.float32(0.37)
    s = np.float32(np.float32(alpha * sa) * sb)
    v = ((av.astype(np.float64) @ bv.astype(np.float64).T).astype(np.float32) * s).astype(np.float32)
    ref = O.e4m3_encode((v * sd).astype(np.float32))
    got, amax = _fp8out(a, b, float(alpha), float(sa), float(sb), float(sd), guard=64)
    assert np.array_equal(got[:M * N].reshape(M, N), ref)
    assert np.all(got[M * N:] == 0xAA)               # nothing written past the matrix
    assert amax == float(np.abs(v).max())


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (200, 136, 4096)])
def test_fp8out_seeded_normal_within_one_code(cuda, built_libs, M, N, K):
    # random data: the tensor-core sum differs from fp64 in the last bits, so a value near a rounding boundary may
    # land on the neighbouring code; never further, and rarely
    cfg = f"fp8out{M}x{N}x{K}"
    a, sa, _ = O.quantize_f32(O.seeded_normal("A", (M, K), config=cfg))
    b, sb, _ = O.quantize_f32(O.seeded_normal("B", (N, K), config=cfg))
    v = O.gemm_f64(a, b, float(np.float32(sa) * np.float32(sb)))
    amax_ref = np.abs(v).max()
    sd = np.float32(448.0 / (1.1 * amax_ref))         # delayed scaling: a slightly stale amax
    ref = O.e4m3_encode((v * float(sd)).astype(np.float32))
    got, amax = _fp8out(a, b, 1.0, float(sa), float(sb), float(sd))
    got = got.reshape(M, N)
    assert abs(amax - amax_ref) <= 1e-5 * amax_ref * np.sqrt(K)
    differ = got != ref
    assert differ.mean() < 5e-3, differ.mean()
    gi, ri = got[differ].astype(np.int32), ref[differ].astype(np.int32)
    assert np.all((np.abs(gi - ri) == 1) | ((gi & 0x7F) + (ri & 0x7F) <= 1))   # neighbours, or +-0 / smallest subnormal


def test_fp8out_saturates_and_amax_optional(cuda, built_libs):
    M, N, K = 128, 64, 64
    a = np.full((M, K), 0x40, np.uint8)              # 2.0
    b = np.full((N, K), 0x40, np.uint8)
    b[1::2] = 0xC0                                   # -2.0
    got, amax = _fp8out(a, b, 1.0, 1.0, 1.0, 1e6, want_amax=False)
    got = got.reshape(M, N)
    assert np.all(got[:, 0::2] == 0x7E) and np.all(got[:, 1::2] == 0xFE)      # +-448, never NaN
    assert amax == 123.0                              # not asked for: not written


def test_tile_pairs_equal_single_tiles_in_every_mode(cuda, built_libs):
    # large problems run as 256-row tile pairs (two accumulators fed from each B tile); fp8_gemm_set_tile_pairs(0) keeps single
    # tiles.  Same MMAs in the same order per output element -> identical bits, in all four epilogues; and sampled rows
    # of the plain result are checked against the restatement.  M = 4224 is 33 row tiles: the last pair is half empty.
    from goml_b200 import fp8_gemm as G
    M, N, K, F = 4224, 19456, 2048, 9728
    g = torch.Generator(device="cuda").manual_seed(7)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.5).to(torch.float8_e4m3fn)
    x0 = torch.randn(M, N, device="cuda", generator=g)
    s = torch.tensor([0.02, 0.5, 3.0], device="cuda")

    def run_all():
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4, G.OutBF16, 0)
        x = x0.clone()
        G.FP8GEMMAccumulateF32(M, N, K, a.data_ptr(), b.data_ptr(), x.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4)
        h = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
        am = torch.zeros(2, device="cuda")
        G.FP8GEMMSwiGLU(M, F, K, a.data_ptr(), b.data_ptr(), h.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4, am.data_ptr())
        d = torch.empty(M, N, dtype=torch.uint8, device="cuda")
        G.FP8GEMMFP8Out(M, N, K, a.data_ptr(), b.data_ptr(), d.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4, s.data_ptr() + 8, am.data_ptr() + 4)
        torch.cuda.synchronize()
        assert G.device_status() == 0
        return c, x, h, d, am

    pair = run_all()
    G.SetTilePairs(0)
    try:
        single = run_all()
    finally:
        G.SetTilePairs(-1)
    for name, p_, s_ in zip(("bf16", "accumulate", "swiglu", "e4m3", "amax"), pair, single):
        assert torch.equal(p_.view(torch.uint8) if p_.dtype != torch.uint8 else p_, s_.view(torch.uint8) if s_.dtype != torch.uint8 else s_), name
    rows = np.array([0, 127, 128, 255, 256, 2047, 4095, 4096, 4200, 4223])
    ah, bh = a.view(torch.uint8).cpu().numpy(), b.view(torch.uint8).cpu().numpy()
    ref = O.gemm_f64(ah[rows], bh, float(np.float32(0.02) * np.float32(0.5)))
    got = pair[0][torch.from_numpy(rows).cuda()].double().cpu().numpy()
    rms = float(np.sqrt(np.mean(ref ** 2)))
    maxabs, meanrel = O.error_stats(got / rms, ref / rms)
    assert maxabs <= 2e-2 and meanrel <= 1e-2, (maxabs, meanrel)


def _device_codes(shape, seed, std=0.5):
    """Seeded e4m3 codes generated on the device (Philox); the same bytes are copied back for the oracle."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * std).to(torch.float8_e4m3fn)


# the shapes the headline numbers are quoted on (8192^3, 16384^3: 256-row tile pairs, 64 / 128 k-blocks through the
# three-stage ring), the shape the one-wave-of-pairs rule exists for (4096 x 4096 x 8192), and pair counts just above a
# multiple of the SM count (150 and 297 pairs on 148 SMs), where single tiles must be chosen instead
@pytest.mark.parametrize("M,N,K", [(8192, 8192, 8192), (16384, 16384, 16384), (4096, 4096, 8192), (2560, 3840, 8192),
                                   (6912, 2816, 2048), (1024, 1024, 1024), (2048, 2048, 2048)])
def test_headline_and_sweep_shapes_on_sampled_rows(cuda, built_libs, M, N, K):
    from goml_b200 import fp8_gemm as G
    a, b = _device_codes((M, K), 100 + M), _device_codes((N, K), 200 + N)
    s = torch.tensor([0.02, 0.5], device="cuda")
    alpha = float(np.float32(0.02) * np.float32(0.5))

    def run():
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4, G.OutBF16, 0)
        torch.cuda.synchronize()
        assert G.device_status() == 0
        return c

    c = run()
    assert torch.isfinite(c).all()
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, M - 129, M - 128, M - 1],
                                     np.random.default_rng(M + N).integers(0, M, 32)]))
    ah, bh = a.view(torch.uint8)[torch.from_numpy(rows).cuda()].cpu().numpy(), b.view(torch.uint8).cpu().numpy()
    check(c[torch.from_numpy(rows).cuda()].double().cpu().numpy(), O.gemm_f64(ah, bh, alpha), True)
    # single tiles give the same bits whichever way the default went
    G.SetTilePairs(0)
    try:
        c1 = run()
    finally:
        G.SetTilePairs(-1)
    assert torch.equal(c.view(torch.int16), c1.view(torch.int16))
    # size-independent: a checksum over every element — column sums of C equal (sum of A's rows) . B^T
    colsum = c.double().sum(0).cpu().numpy()
    a_sum = O.e4m3_decode(a.view(torch.uint8).cpu().numpy()).astype(np.float64).sum(0)
    want = (O.e4m3_decode(bh).astype(np.float64) @ a_sum) * alpha
    # each bf16 element carries a rounding error of std ~2.3e-3 |c| with random sign: six standard deviations of the sum
    # (a missing 128-row tile would be off by ~128 r_elem, a hundred times the bound)
    r_elem = float(c.double().pow(2).mean().sqrt().item())
    assert np.abs(colsum - want).max() <= 1.4e-2 * np.sqrt(M) * r_elem


@pytest.mark.parametrize("M", [16, 128])
def test_skinny_shapes_in_full(cuda, built_libs, M):
    # M in {16, 128}, N = K = 8192: HBM-bound shapes of the sweep (narrow tiles, two k-blocks per stage, 32 stages deep;
    # split over K in accumulate mode), every element against the oracle
    from goml_b200 import fp8_gemm as G
    N = K = 8192
    a, b = _device_codes((M, K), 300 + M), _device_codes((N, K), 301 + M)
    s = torch.tensor([0.03, 0.25], device="cuda")
    alpha = float(np.float32(0.03) * np.float32(0.25))
    ref = O.gemm_f64(a.view(torch.uint8).cpu().numpy(), b.view(torch.uint8).cpu().numpy(), alpha)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4, G.OutBF16, 0)
    x0 = torch.randn(M, N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    x = x0.clone()
    G.FP8GEMMAccumulateF32(M, N, K, a.data_ptr(), b.data_ptr(), x.data_ptr(), 1.0, s.data_ptr(), s.data_ptr() + 4)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    check(c.double().cpu().numpy(), ref, True)
    rms = float(np.sqrt(np.mean(ref ** 2)))
    err = np.abs(x.double().cpu().numpy() - (x0.double().cpu().numpy() + ref)).max()
    assert err <= 1e-5 * max(rms, 1.0) * np.sqrt(K), err
