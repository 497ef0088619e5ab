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
