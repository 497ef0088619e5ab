"""Quantiser parity on the GPU: e4m3 codes, scale and amax bit-exact against the oracle."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def gpu_quant(x, convention):
    from goml_b200 import quantize as Q
    xd = torch.from_numpy(np.ascontiguousarray(x, np.float32).ravel()).cuda()
    q = torch.full((xd.numel() + 16,), 0xAA, dtype=torch.uint8, device="cuda")
    sa = torch.full((2,), 123.0, dtype=torch.float32, device="cuda")  # stale amax/scale must not matter
    fn = Q.QuantizeF32ToF8E4M3Unit if convention == 1 else Q.QuantizeF32ToF8E4M3
    fn(xd.data_ptr(), q.data_ptr(), sa.data_ptr(), sa.data_ptr() + 4, xd.numel(), 0)
    torch.cuda.synchronize()
    assert torch.all(q[xd.numel():] == 0xAA)  # nothing written past n
    return q[: xd.numel()].cpu().numpy().reshape(np.shape(x)), np.float32(sa[0].item()), np.float32(sa[1].item())


@pytest.mark.parametrize("convention", [0, 1])
@pytest.mark.parametrize("n", [1, 15, 16, 17, 1000, 4096 * 33 + 5, 1 << 22])
def test_codes_bit_exact(cuda, built_libs, convention, n):
    x = O.seeded_normal("x", (n,), std=1.0 if n % 2 else 0.02, config=f"q{n}")
    q, scale, amax = gpu_quant(x, convention)
    wq, wscale, wamax = O.quantize_f32(x, convention)
    assert amax == wamax and scale == wscale
    assert np.array_equal(q, wq)


def test_special_values(cuda, built_libs):
    x = O.seeded_normal("x", (4099,), config="special")
    x[7] = np.nan
    x[100] = -0.0
    x[200] = 1e-30
    x[300] = 17.5   # becomes amax
    q, scale, amax = gpu_quant(x, 0)
    wq, wscale, wamax = O.quantize_f32(x, 0)
    assert amax == wamax == 17.5 and scale == wscale
    assert np.array_equal(q, wq)
    z = np.zeros(64, np.float32)
    q, scale, amax = gpu_quant(z, 0)
    assert scale == 1.0 and amax == 0.0 and not q.any()


def test_attention_shaped_tensor_both_conventions(cuda, built_libs):
    x = O.seeded_normal("Q", (4, 256, 64), config="C1")
    for conv in (0, 1):
        q, scale, _ = gpu_quant(x, conv)
        wq, wscale, _ = O.quantize_f32(x, conv)
        assert scale == wscale and np.array_equal(q, wq)


def test_dequantize_roundtrip(cuda, built_libs):
    from goml_b200 import quantize as Q
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    qd = torch.from_numpy(codes).cuda()
    out = torch.empty(codes.size, dtype=torch.float16, device="cuda")
    s = torch.tensor([0.5], dtype=torch.float32, device="cuda")
    Q.DequantizeToFP16(qd.data_ptr(), out.data_ptr(), s.data_ptr(), codes.size)
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), O.e4m3_decode(codes) * 0.5)


@pytest.mark.parametrize("n", [1, 2, 7, 1000, 1023, 4096 * 33 + 5, 1 << 22])
def test_codes_and_scale_equal_the_reference_quantiser_kernel(cuda, built_libs, n):
    # north_star: "bit-exact match on e4m3 quantisation codes" with the reference.  The reference's own quantiser
    # (libs1/fp8_quantize_v2.cu:176-204, built for this GPU as it stands into oracle/_ref/libref_quant.so) and
    # this library's fp8_quantize_fp16 get the same FP16 tensor; fp8_quantize_f32 gets the same values as FP32.
    from goml_b200 import quantize as Q
    R = O.ref()
    if R.quant is None:
        pytest.skip("oracle/_ref/libref_quant.so was not built (the reference tree was absent at build time)")
    x = O.seeded_normal("x", (n,), std=3.0 if n % 2 else 0.02, config=f"qref{n}").astype(np.float16)
    xd = torch.from_numpy(x).cuda()
    want = torch.full((n + 16,), 0xAA, dtype=torch.uint8, device="cuda")
    wscale = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert R.quant.fp8_quantize_fp16(xd.data_ptr(), want.data_ptr(), wscale.data_ptr(), n) == 0
    assert R.quant.cuda_device_sync2() == 0
    got = torch.full((n + 16,), 0xAA, dtype=torch.uint8, device="cuda")
    gscale = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")
    Q.QuantizeFP16(xd.data_ptr(), got.data_ptr(), gscale.data_ptr(), n)
    Q.DeviceSync2()
    assert gscale.item() == wscale.item()
    assert torch.equal(got, want)                       # codes, and nothing written past n by either
    # the FP32 entry on the same (fp16-representable) values: same codes, same scale
    x32 = torch.from_numpy(x.astype(np.float32)).cuda()
    q32 = torch.empty(n, dtype=torch.uint8, device="cuda")
    sa = torch.zeros(2, dtype=torch.float32, device="cuda")
    Q.QuantizeF32ToF8E4M3(x32.data_ptr(), q32.data_ptr(), sa.data_ptr(), sa.data_ptr() + 4, n, 0)
    torch.cuda.synchronize()
    assert sa[0].item() == wscale.item() and torch.equal(q32, want[:n])
    # and the CPU restatement agrees with all three
    oq, oscale, _ = O.quantize_f32(x.astype(np.float32), 0)
    assert np.float32(wscale.item()) == oscale and np.array_equal(want[:n].cpu().numpy(), oq)
