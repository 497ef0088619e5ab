"""FP8 attention-forward parity on the GPU, through the C ABI, against the oracle.

Tolerance (stated bar): max-abs error <= 2e-2 and mean relative error
(mean|x-ref| / mean|ref|) <= 1e-2 on the fp16 output, against the fp64 oracle on
the same e4m3 codes.  The reference's own gates are also applied where its
tests define them: |gpu-cpu| <= max(0.05, 0.1|cpu|) on its eight self-check
shapes (libs/flash_attention_v121r_diet_hd128_fp8_forward.cu:1026), LSE within
5e-3 relative (backend/cuda/fa_forward_test.go:186) and O/L within 5e-3 absolute
of a CPU-F64 loop (backend/cuda/fa_chain_cpuref_test.go:268).
"""
import math

import numpy as np
import pytest
import torch

import oracle as O
from tests.golden.make_golden import ATTN_SHAPES
from tests.gpu_util import dev_u8, run_attention

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 2e-2, 1e-2


def check(o, ref, lse=None, lse_ref=None):
    maxabs, meanrel = O.error_stats(o, ref)
    assert maxabs <= MAX_ABS, maxabs
    assert meanrel <= MEAN_REL, meanrel
    if lse is not None:
        fin = np.isfinite(lse_ref)
        assert np.array_equal(np.isfinite(lse), fin)
        assert np.abs(lse[fin] - lse_ref[fin]).max() <= 5e-3


@pytest.mark.parametrize("name", sorted(ATTN_SHAPES))
def test_reference_selfcheck_shapes(fa_ctx, golden, name):
    bh, sl, hd, ca, w = ATTN_SHAPES[name]
    q, k, v = O.harness_attention_inputs(bh, sl, hd)
    o, lse = run_attention(fa_ctx, q, k, v, ca, w)
    ref = golden[f"attn_{name}_o"].astype(np.float64)         # the reference's own cpu_attention_fp8
    assert np.all(np.abs(o - ref) <= np.maximum(0.05, 0.1 * np.abs(ref)))   # the reference's gate
    o64, l64 = O.attention_f64(q, k, v, ca, w)
    check(o, o64, lse, l64)


@pytest.mark.parametrize("conv", [0, 1])
@pytest.mark.parametrize("entry", ["train", "forward", "ex"])
def test_config1(fa_ctx, conv, entry):
    # B=1, H=4, S=256, D=64, non-causal, N(0,1) quantised per tensor (amax/448 and amax), scale 1/sqrt(64)
    qs = [O.quantize_f32(O.seeded_normal(n, (4, 256, 64), config="C1"), conv) for n in "QKV"]
    (q, sq, _), (k, sk, _), (v, sv, _) = qs
    scale = float(sq) * float(sk) / math.sqrt(64)
    if entry == "ex":
        o, lse = run_attention(fa_ctx, q, k, v, 0, 0, scale, v_descale=float(sv), entry="ex")
        ref, lref = O.attention_f64(q, k, v, 0, 0, scale, float(sv))
    else:
        # reference convention: O in decoded-V units, the caller multiplies by scale_V in fp32
        o, lse = run_attention(fa_ctx, q, k, v, 0, 0, scale, entry=entry)
        o = o * float(sv)
        ref, lref = O.attention_f64(q, k, v, 0, 0, scale, float(sv))
    check(o, ref, lse, lref if lse is not None else None)
    # and against the reference's fp32 CPU arithmetic (backend/cpu/cpu.go:394-461) on the same codes
    if conv == 1:
        o32 = O.attention_f32(q, k, v, 0, 0, np.float32(scale), parallel=True).astype(np.float64) * float(sv)
        check(o, o32)


CASES = [
    # bh, sl, hd, causal, window
    (1, 1, 128, 0, 0), (1, 1, 64, 1, 0), (2, 17, 128, 1, 0), (3, 280, 128, 0, 0), (2, 300, 64, 1, 0),
    (1, 129, 128, 1, 0), (1, 127, 64, 0, 0), (2, 1000, 128, 1, 200), (2, 1000, 64, 0, 333),
    (1, 512, 128, 1, 1), (1, 512, 64, 1, 512), (4, 1024, 128, 0, 0), (4, 1024, 64, 1, 0), (1, 2048, 128, 1, 128),
    # more heads than one group of the causal / window tile order (groups of 16 heads, longest tiles first), last group partial
    (19, 300, 128, 1, 0), (37, 260, 64, 1, 50), (33, 257, 128, 0, 100),
]


@pytest.mark.parametrize("bh,sl,hd,ca,w", CASES)
def test_ragged_masks_windows(fa_ctx, bh, sl, hd, ca, w):
    cfg = f"fa{bh}_{sl}_{hd}_{ca}_{w}"
    (q, sq, _), (k, sk, _), (v, sv, _) = [O.quantize_f32(O.seeded_normal(n, (bh, sl, hd), config=cfg), 0) for n in "QKV"]
    scale = float(sq) * float(sk) / math.sqrt(hd)
    o, lse = run_attention(fa_ctx, q, k, v, ca, w, scale, v_descale=float(sv), entry="ex")
    ref, lref = O.attention_f64(q, k, v, ca, w, scale, float(sv))
    check(o, ref, lse, lref)


@pytest.mark.parametrize("scale_sign", [-1.0, 0.0])
def test_negative_and_zero_scale(fa_ctx, scale_sign):
    # the scale is a free float in the ABI: a negative one reverses the ranking of the keys, zero gives uniform weights
    bh, sl, hd = 2, 300, 128
    (q, sq, _), (k, sk, _), (v, sv, _) = [O.quantize_f32(O.seeded_normal(n, (bh, sl, hd), config="negscale"), 0) for n in "QKV"]
    scale = scale_sign * float(sq) * float(sk) / math.sqrt(hd)
    for causal in (0, 1):
        o, lse = run_attention(fa_ctx, q, k, v, causal, 0, scale, v_descale=float(sv), entry="ex")
        ref, lref = O.attention_f64(q, k, v, causal, 0, scale, float(sv))
        check(o, ref, lse, lref)


def test_lse_uniform_and_layout(fa_ctx):
    # backend/cuda/fa_forward_test.go:112-189 and :191-288
    bh, sl, hd = 3, 280, 128
    ones = np.full((bh, sl, hd), 0x38, np.uint8)
    o, lse = run_attention(fa_ctx, ones, ones, ones)
    want = math.sqrt(hd) + math.log(sl)
    assert np.abs(lse - want).max() / want <= 5e-3
    assert np.allclose(o, 1.0, atol=1e-3)
    qh = np.stack([np.full((sl, hd), c, np.uint8) for c in (0x38, 0x40, 0x48)])
    _, lse = run_attention(fa_ctx, qh, ones, ones)
    for i in range(3):
        want = 2 ** i * math.sqrt(hd) + math.log(sl)
        assert np.abs(lse[i] - want).max() / want <= 5e-3   # rows of head i, i.e. a [bh, sl] layout


def test_magnitude_contract_properties(fa_ctx):
    # backend/cuda/fa_contract_test.go:188-279: decoded |x| <= 1 codes with random sign
    rng = np.random.default_rng(321)
    bh, sl, hd = 4, 2048, 128
    pool = np.array([c for c in range(0x78) if O.e4m3_decode(np.uint8(c)) <= 1.0], np.uint8)

    def draw():
        return pool[rng.integers(0, pool.size, (bh, sl, hd))] | (rng.integers(0, 2, (bh, sl, hd), dtype=np.uint8) << 7)

    q, k, v = draw(), draw(), draw()
    scale = 1.0 / math.sqrt(hd)
    o, lse = run_attention(fa_ctx, q, k, v, 0, 0, scale)
    assert np.isfinite(o).all() and np.isfinite(lse).all()
    assert lse.max() <= scale * hd * 1.0 + math.log(sl) + 1e-3          # L <= scale*hd*max^2 + ln sl
    v2 = v.copy()
    v2[:, 5, :] ^= 0x08                                                  # flip one mantissa/exponent bit of one V row
    o2, _ = run_attention(fa_ctx, q, k, v2, 0, 0, scale)
    assert np.abs(o2 - o).max() > 0
    ref, lref = O.attention_f64_rows(q, k, v, 1000, 1032, 0, 0, scale)
    check(o[:, 1000:1032], ref, lse[:, 1000:1032], lref)


def test_chain_vs_cpu_f64(fa_ctx):
    # backend/cuda/fa_chain_cpuref_test.go:48-75,268-286: bh1/sl128/hd128, floor 5e-3 abs on O and L
    rng = np.random.default_rng(101)
    x = [(rng.random((1, 128, 128), dtype=np.float32) * 2 - 1) for _ in range(3)]
    (q, sq, _), (k, sk, _), (v, sv, _) = [O.quantize_f32(t, 1) for t in x]
    scale = float(sq) * float(sk) / math.sqrt(128)
    o, lse = run_attention(fa_ctx, q, k, v, 1, 0, scale)
    ref, lref = O.attention_f64(q, k, v, 1, 0, scale)
    assert np.abs(o - ref).max() <= 5e-3 and np.abs(lse - lref).max() <= 5e-3


def test_argument_validation(fa_ctx):
    from goml_b200 import fa_forward as F
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()

    def status(fn, *a):
        with pytest.raises(F.FAError) as e:
            fn(*a)
        return e.value.status, str(e.value)

    s, msg = status(fa_ctx.ForwardTrain, 0, p, p, p, 0, 1, 64, 128, 0, 0, 1.0)
    assert s == F.FA_ERR_INVALID_ARG and "null pointer" in msg
    assert status(fa_ctx.ForwardTrain, p, p, p, p, 0, 0, 64, 128, 0, 0, 1.0)[0] == F.FA_ERR_INVALID_ARG
    assert status(fa_ctx.ForwardTrain, p, p, p, p, 0, 1, 64, 96, 0, 0, 1.0)[0] == F.FA_ERR_UNSUPPORTED_HD
    assert status(fa_ctx.ForwardTrain, p, p, p, p, 0, 1, 64, 128, 0, 65, 1.0)[0] == F.FA_ERR_INVALID_ARG
    assert status(fa_ctx.ForwardTrain, p, p, p, p, 0, 1, 64, 128, 2, 0, 1.0)[0] == F.FA_ERR_INVALID_ARG
    assert status(fa_ctx.Forward, p + 1, p, p, p, 1, 64, 128, 0, 0, 1.0)[0] == F.FA_ERR_INVALID_ARG
    fa_ctx.ForwardTrain(p, p, p, p + 32768, 0, 1, 64, 128, 0, 0, 1.0)   # NULL l_out is allowed
    torch.cuda.synchronize()
    fa_ctx.DeviceStatus()


def test_offset_subbuffers_and_other_allocators(fa_ctx):
    # pointers that are views into a larger allocation (pool sub-buffers), 256-byte aligned like backend/cuda/pool.go:52-56
    bh, sl, hd = 2, 192, 128
    q, k, v = O.harness_attention_inputs(bh, sl, hd)
    n = bh * sl * hd
    arena = torch.zeros(4 * n + 4096, dtype=torch.uint8, device="cuda")
    offs = [256, 256 + n + 768, 256 + 2 * n + 1792]
    for src, off in zip((q, k, v), offs):
        arena[off:off + n] = dev_u8(src).ravel()
    o = torch.zeros((bh, sl, hd), dtype=torch.float16, device="cuda")
    base = arena.data_ptr()
    fa_ctx.ForwardTrain(base + offs[0], base + offs[1], base + offs[2], o.data_ptr(), 0, bh, sl, hd, 1, 0, 1 / math.sqrt(hd))
    torch.cuda.synchronize()
    ref, _ = O.attention_f64(q, k, v, 1, 0)
    check(o.double().cpu().numpy(), ref)


@pytest.mark.parametrize("causal", [0, 1])
def test_config3_full_size_sampled(fa_ctx, causal):
    # B=4, H=32 (BH=128), S=8192, D=128, fp16 O + fp32 LSE; oracle on sampled heads x row blocks
    bh, sl, hd = 128, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(1234)
    x = [torch.randn((bh, sl, hd), generator=g, device="cuda") for _ in range(3)]
    from goml_b200 import quantize as Q
    codes, scales = [], torch.zeros(6, dtype=torch.float32, device="cuda")
    for i, t in enumerate(x):
        c = torch.empty((bh, sl, hd), dtype=torch.uint8, device="cuda")
        Q.QuantizeF32ToF8E4M3(t.data_ptr(), c.data_ptr(), scales.data_ptr() + 8 * i, scales.data_ptr() + 8 * i + 4, t.numel(), 0)
        codes.append(c)
    del x
    o = torch.zeros((bh, sl, hd), dtype=torch.float16, device="cuda")
    lse = torch.zeros((bh, sl), dtype=torch.float32, device="cuda")
    q, k, v = codes
    fa_ctx.ForwardEx(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), bh, sl, hd, causal, 0,
                     1.0 / math.sqrt(hd), 1.0, scales.data_ptr(), scales.data_ptr() + 8, scales.data_ptr() + 16)
    torch.cuda.synchronize()
    fa_ctx.DeviceStatus()
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    sc = scales.cpu().numpy()
    scale = float(sc[0]) * float(sc[2]) / math.sqrt(hd)
    for h, r0 in [(0, 0), (37, 4096 - 16), (127, 8192 - 32)]:
        qh, kh, vh = (t[h:h + 1].cpu().numpy() for t in (q, k, v))
        ref, lref = O.attention_f64_rows(qh, kh, vh, r0, r0 + 32, causal, 0, scale, float(sc[4]))
        check(o[h:h + 1, r0:r0 + 32].double().cpu().numpy(), ref,
              lse[h:h + 1, r0:r0 + 32].double().cpu().numpy(), lref)
    # size-independent properties: heads are independent (a copy of head 5's data placed at head 9 gives
    # identical bits), and the result does not depend on which other heads are in the batch
    for t in (q, k, v):
        t[9] = t[5]
    o2 = torch.zeros_like(o[:16])
    fa_ctx.ForwardEx(q.data_ptr(), k.data_ptr(), v.data_ptr(), o2.data_ptr(), 0, 16, sl, hd, causal, 0,
                     1.0 / math.sqrt(hd), 1.0, scales.data_ptr(), scales.data_ptr() + 8, scales.data_ptr() + 16)
    torch.cuda.synchronize()
    assert torch.equal(o2[9], o2[5]) and torch.equal(o2[5], o[5])


# the long-sequence cells of the sweep (B*S = 65536 tokens, H = 32): 64-bit indexing, grids of 16384 CTAs
@pytest.mark.parametrize("causal", [0, 1])
@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("bh,sl", [(128, 16384), (64, 32768), (512, 4096), (2048, 1024)])
def test_sweep_cells_on_sampled_blocks(fa_ctx, bh, sl, hd, causal):
    # inputs drawn on the device from a fixed Philox seed and quantised there; the same code bytes and scales are copied
    # back for the oracle, which is evaluated on three (head, 32-row) blocks
    from goml_b200 import quantize as Q
    g = torch.Generator(device="cuda").manual_seed(bh * 7 + sl + hd)
    codes, scales = [], torch.zeros(6, dtype=torch.float32, device="cuda")
    for i in range(3):
        t = torch.randn((bh, sl, hd), generator=g, device="cuda")
        c = torch.empty((bh, sl, hd), dtype=torch.uint8, device="cuda")
        Q.QuantizeF32ToF8E4M3(t.data_ptr(), c.data_ptr(), scales.data_ptr() + 8 * i, scales.data_ptr() + 8 * i + 4, t.numel(), 0)
        torch.cuda.synchronize()
        del t
        codes.append(c)
    q, k, v = codes
    o = torch.zeros((bh, sl, hd), dtype=torch.float16, device="cuda")
    lse = torch.zeros((bh, sl), dtype=torch.float32, device="cuda")
    fa_ctx.ForwardEx(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), bh, sl, hd, causal, 0,
                     1.0 / math.sqrt(hd), 1.0, scales.data_ptr(), scales.data_ptr() + 8, scales.data_ptr() + 16)
    torch.cuda.synchronize()
    fa_ctx.DeviceStatus()
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    sc = scales.cpu().numpy()
    scale = float(sc[0]) * float(sc[2]) / math.sqrt(hd)
    for h, r0 in [(0, 0), (bh // 3, sl // 2 - 16), (bh - 1, sl - 32)]:
        qh, kh, vh = (t[h:h + 1].cpu().numpy() for t in (q, k, v))
        ref, lref = O.attention_f64_rows(qh, kh, vh, r0, r0 + 32, causal, 0, scale, float(sc[4]))
        check(o[h:h + 1, r0:r0 + 32].double().cpu().numpy(), ref,
              lse[h:h + 1, r0:r0 + 32].double().cpu().numpy(), lref)
    # size-independent property over every row: softmax weights sum to one, so with V replaced by the code of 1.0
    # every output element is v_descale (here 1) whatever Q and K hold
    v.fill_(0x38)
    fa_ctx.ForwardEx(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 0, bh, sl, hd, causal, 0,
                     1.0 / math.sqrt(hd), 1.0, scales.data_ptr(), scales.data_ptr() + 8, 0)
    torch.cuda.synchronize()
    fa_ctx.DeviceStatus()
    assert (o.float() - 1.0).abs().max().item() <= 2e-3
