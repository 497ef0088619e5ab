"""Decoder-block glue fused with the quantiser (libfp8block.so) against the numpy restatement.

Bar: e4m3 codes bit-exact wherever the fp32 operation order is fully specified (RoPE + permute of Q/K/V,
head permute of the attention output: the products and the single add are individually rounded on both
sides).  RMSNorm sums squares in a different order and SwiGLU uses the device's expf, so there the
quantiser INPUT can differ in the last fp32 bit: scales must agree to 1e-6 relative, at most 1e-4 of
the codes may differ, and every difference is one code step.
"""
import numpy as np
import pytest
import torch

import oracle as O
from oracle import glue

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def code_steps(a, b):
    """Distance in e4m3 code steps between two code arrays (sign-magnitude ordering)."""
    def key(c):
        c = c.astype(np.int32)
        return np.where(c & 0x80, -(c & 0x7f), c & 0x7f)
    return np.abs(key(a) - key(b))


def nearly_same_codes(got, want, frac=1e-4):
    steps = code_steps(got, want)
    assert steps.max() <= 1, steps.max()
    assert (steps != 0).mean() <= frac, (steps != 0).mean()


@pytest.mark.parametrize("rows,hidden,with_res", [(96, 512, False), (300, 4096, True), (2500, 4096, False), (64, 2048, False), (40, 8192, True), (7, 1040, True), (0, 64, False)])
def test_rmsnorm_quantize(cuda, built_libs, rows, hidden, with_res):
    from goml_b200 import block_glue as BG
    cfg = f"rms{rows}_{hidden}"
    x = O.seeded_normal("x", (rows, hidden), config=cfg).astype(np.float32)
    res = glue.bf16_values(0.5 * O.seeded_normal("r", (rows, hidden), config=cfg)) if with_res else None
    gamma = (1.0 + 0.1 * O.seeded_normal("g", (hidden,), config=cfg)).astype(np.float32)
    xd = dev(x) if rows else torch.zeros(16, device="cuda")
    rd = dev(res, torch.bfloat16) if with_res else None
    q = torch.full((max(rows, 1), hidden), 0xAA, dtype=torch.uint8, device="cuda")
    sa = torch.full((2,), 7.0, dtype=torch.float32, device="cuda")
    rstd = torch.empty(max(rows, 1), dtype=torch.float32, device="cuda")
    gd = dev(gamma)
    BG.RMSNormQuantize(xd.data_ptr(), rd.data_ptr() if with_res else 0, xd.data_ptr() if with_res else 0, gd.data_ptr(),
                       q.data_ptr(), sa.data_ptr(), sa.data_ptr() + 4, rstd.data_ptr(), rows, hidden, 1e-5)
    torch.cuda.synchronize()
    if rows == 0:
        assert sa.tolist() == [1.0, 0.0]
        return
    codes, scale, amax, h, _ = glue.rmsnorm_quantize(x, res, gamma, 1e-5)
    assert abs(sa[0].item() - scale) <= 1e-6 * scale and abs(sa[1].item() - amax) <= 1e-6 * amax
    nearly_same_codes(q.cpu().numpy()[:rows], codes)
    if with_res:  # the residual stream was updated in place, exactly
        assert np.array_equal(xd.cpu().numpy(), h)


@pytest.mark.parametrize("B,S,H,hd", [(2, 64, 4, 128), (1, 200, 3, 64), (3, 33, 2, 128)])
def test_rope_quantize_qkv_bit_exact(cuda, built_libs, B, S, H, hd):
    from goml_b200 import block_glue as BG
    cfg = f"rope{B}_{S}_{H}_{hd}"
    qkv = glue.bf16_values(O.seeded_normal("qkv", (B * S, 3, H, hd), config=cfg) * np.array([1.0, 3.0, 0.25])[None, :, None, None])
    cos = torch.empty((S, hd // 2), dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    BG.RopeTable(cos.data_ptr(), sin.data_ptr(), S, hd, 10000.0)
    c_ref, s_ref = glue.rope_table(S, hd, 10000.0)
    torch.cuda.synchronize()
    assert np.abs(cos.cpu().numpy() - c_ref).max() <= 6e-8 and np.abs(sin.cpu().numpy() - s_ref).max() <= 6e-8
    # feed the kernel the restatement's tables so that the comparison below is bit-exact
    cos, sin = dev(c_ref), dev(s_ref)
    out = [torch.full((B * H, S, hd), 0xAA, dtype=torch.uint8, device="cuda") for _ in range(3)]
    s6 = torch.full((6,), 9.0, dtype=torch.float32, device="cuda")
    qkv_d = dev(qkv, torch.bfloat16)
    BG.RopeQuantizeQKV(qkv_d.data_ptr(), cos.data_ptr(), sin.data_ptr(), out[0].data_ptr(), out[1].data_ptr(),
                       out[2].data_ptr(), s6.data_ptr(), s6.data_ptr() + 12, B, S, H, hd)
    torch.cuda.synchronize()
    want = glue.rope_quantize_qkv(qkv, c_ref, s_ref, B, S, H, hd)
    for w in range(3):
        codes, scale, amax = want[w]
        assert s6[w].item() == scale and s6[3 + w].item() == amax, (w, s6.tolist(), scale, amax)
        assert np.array_equal(out[w].cpu().numpy(), codes), w


@pytest.mark.parametrize("B,S,H,hd", [(2, 64, 4, 128), (1, 50, 3, 64)])
def test_permute_quantize_heads_bit_exact(cuda, built_libs, B, S, H, hd):
    from goml_b200 import block_glue as BG
    o = O.round_fp16(O.seeded_normal("o", (B * H, S, hd), config=f"perm{B}_{S}_{H}_{hd}")).astype(np.float32)
    q = torch.full((B * S, H * hd), 0xAA, dtype=torch.uint8, device="cuda")
    sa = torch.zeros(2, dtype=torch.float32, device="cuda")
    od = dev(o, torch.float16)
    BG.PermuteQuantizeHeads(od.data_ptr(), q.data_ptr(), sa.data_ptr(), sa.data_ptr() + 4, B, S, H, hd)
    torch.cuda.synchronize()
    codes, scale, amax = glue.permute_quantize_heads(o, B, S, H, hd)
    assert sa.tolist() == [scale, amax]
    assert np.array_equal(q.cpu().numpy(), codes)


@pytest.mark.parametrize("rows,F", [(64, 1376), (33, 704), (5, 11008)])
def test_swiglu_quantize(cuda, built_libs, rows, F):
    from goml_b200 import block_glue as BG
    gu = glue.bf16_values(2.0 * O.seeded_normal("gu", (rows, 2 * F), config=f"swiglu{rows}_{F}"))
    q = torch.full((rows, F), 0xAA, dtype=torch.uint8, device="cuda")
    sa = torch.zeros(2, dtype=torch.float32, device="cuda")
    gud = dev(gu, torch.bfloat16)
    BG.SwiGLUQuantize(gud.data_ptr(), q.data_ptr(), sa.data_ptr(), sa.data_ptr() + 4, rows, F)
    torch.cuda.synchronize()
    codes, scale, amax, _ = glue.swiglu_quantize(gu, F)
    assert abs(sa[0].item() - scale) <= 1e-6 * scale and abs(sa[1].item() - amax) <= 1e-6 * amax
    nearly_same_codes(q.cpu().numpy(), codes)


def test_residual_add_exact(cuda, built_libs):
    from goml_b200 import block_glue as BG
    x = O.seeded_normal("x", (1000, 72), config="resadd").astype(np.float32)
    y = glue.bf16_values(O.seeded_normal("y", (1000, 72), config="resadd"))
    xd = dev(x)
    yd = dev(y, torch.bfloat16)
    BG.ResidualAdd(xd.data_ptr(), yd.data_ptr(), x.size)
    torch.cuda.synchronize()
    assert np.array_equal(xd.cpu().numpy(), x + y)


def test_rejects_bad_arguments(cuda, built_libs):
    from goml_b200 import block_glue as BG
    buf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(BG.BlockGlueError):
        BG.RMSNormQuantize(p, 0, 0, p, p, p, p + 4, p, 4, 24, 1e-5)          # hidden not a multiple of 16
    with pytest.raises(BG.BlockGlueError):
        BG.RMSNormQuantize(p + 4, 0, 0, p, p, p, p + 4, p, 4, 32, 1e-5)      # misaligned x
    with pytest.raises(BG.BlockGlueError):
        BG.RopeQuantizeQKV(p, p, p, p, p, p, p, p, 1, 8, 2, 96)              # head_dim 96
    with pytest.raises(BG.BlockGlueError):
        BG.SwiGLUQuantize(p, p, p, p, 2, 40)                                 # ffn_hidden not a multiple of 16
    with pytest.raises(BG.BlockGlueError):
        BG.ResidualAdd(p, p, 12)                                             # n not a multiple of 8
