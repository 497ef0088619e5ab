"""Llama-style decoder block with every GEMM and the attention in FP8 (the block config at reduced
size): product chain (goml_b200.nn) against the CPU restatement with the same quantisation points.

Tolerance: the stated bar (max-abs <= 2e-2, mean relative <= 1e-2) on the block output, and on every
quantised stage run on the restatement's own inputs (there the kernels agree to ~1e-3 or better).
What the whole block ADDS to its input is checked at mean relative <= 5e-2: each re-quantisation turns a
1e-4 difference of its input (fp16 rounding of the attention output) into isolated e4m3 code flips,
which the following GEMM spreads — measured growth about 10x per stage, a property of per-tensor FP8
chains, not of the kernels (the o-projection fed the restatement's input agrees to 1e-11).
"""
import numpy as np
import pytest
import torch

import oracle as O
from oracle.decoder_block import decoder_block

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("B,S,d,H,Fh", [(2, 256, 512, 4, 1376), (1, 384, 256, 4, 704)])
def test_block_matches_cpu_restatement(cuda, built_libs, B, S, d, H, Fh, fused):
    from goml_b200 import nn
    cfg = f"block{B}_{S}_{d}"
    w = {n: O.seeded_normal(n, shp, std=0.02, config=cfg) for n, shp in
         dict(wqkv=(3 * d, d), wo=(d, d), wgate_up=(2 * Fh, d), wdown=(d, Fh)).items()}
    g1 = 1.0 + 0.1 * O.seeded_normal("g1", (d,), config=cfg)
    g2 = 1.0 + 0.1 * O.seeded_normal("g2", (d,), config=cfg)
    x = O.seeded_normal("x", (B * S, d), config=cfg)
    t = lambda a: torch.from_numpy(a).cuda()
    blk = nn.FP8DecoderBlock(d, H, Fh, t(w["wqkv"]), t(w["wo"]), t(w["wgate_up"]), t(w["wdown"]), t(g1.astype(np.float32)), t(g2.astype(np.float32)), fused=fused)
    y = blk(t(x), B, S)
    torch.cuda.synchronize()
    blk.fa.DeviceStatus()
    blk.close()
    got = y.double().cpu().numpy()
    ref = decoder_block(x, B, S, H, w["wqkv"], w["wo"], w["wgate_up"], w["wdown"], g1, g2, residual_in_epilogue=fused, swiglu_in_epilogue=fused)
    assert np.isfinite(got).all()
    maxabs, meanrel = O.error_stats(got, ref)
    assert maxabs <= 2e-2 and meanrel <= 1e-2, (maxabs, meanrel)
    maxabs_d, meanrel_d = O.error_stats(got - x, ref - x)
    assert maxabs_d <= 2e-2 and meanrel_d <= 5e-2, (maxabs_d, meanrel_d)


def test_each_stage_on_identical_inputs(cuda, built_libs):
    from goml_b200 import nn
    B, S, d, H, Fh = 2, 256, 512, 4, 1376
    cfg = "block-stages"
    w = {n: O.seeded_normal(n, shp, std=0.02, config=cfg) for n, shp in
         dict(wqkv=(3 * d, d), wo=(d, d), wgate_up=(2 * Fh, d), wdown=(d, Fh)).items()}
    g = np.ones(d)
    x = O.seeded_normal("x", (B * S, d), config=cfg)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    blk = nn.FP8DecoderBlock(d, H, Fh, t(w["wqkv"]), t(w["wo"]), t(w["wgate_up"]), t(w["wdown"]), t(g), t(g))
    inter = {}
    decoder_block(x, B, S, H, w["wqkv"], w["wo"], w["wgate_up"], w["wdown"], g, g, intermediates=inter)

    def close(got, ref, tol=(2e-2, 1e-2)):
        maxabs, meanrel = O.error_stats(got.double().cpu().numpy(), ref)
        assert maxabs <= tol[0] and meanrel <= tol[1], (maxabs, meanrel)

    close(nn.rms_norm(t(x), blk.norm1, blk.eps), inter["xn1"], (1e-5, 1e-6))
    close(blk.qkv(t(inter["xn1"])), inter["qkv"], (2e-2, 1e-4))          # same codes -> same bf16 values
    close(blk.attention(t(inter["xn1"]), B, S), inter["attn"], (2e-2, 2e-3))
    close(blk.o(t(inter["attn"])), inter["ao"], (2e-2, 1e-4))
    close(blk.gate_up(t(inter["xn2"])), inter["gu"], (2e-2, 1e-4))
    close(blk.down(t(inter["h"])), inter["ffn"], (2e-2, 1e-4))
    torch.cuda.synchronize()
    blk.fa.DeviceStatus()
    blk.close()


def _make_block(cfg, d, H, Fh):
    from goml_b200 import nn
    w = {n: O.seeded_normal(n, shp, std=0.02, config=cfg) for n, shp in
         dict(wqkv=(3 * d, d), wo=(d, d), wgate_up=(2 * Fh, d), wdown=(d, Fh)).items()}
    g1 = 1.0 + 0.1 * O.seeded_normal("g1", (d,), config=cfg)
    g2 = 1.0 + 0.1 * O.seeded_normal("g2", (d,), config=cfg)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    blk = nn.FP8DecoderBlock(d, H, Fh, t(w["wqkv"]), t(w["wo"]), t(w["wgate_up"]), t(w["wdown"]), t(g1), t(g2))
    return blk, w, g1, g2, t


@pytest.mark.parametrize("B,d,H,Fh,Smax", [(3, 512, 4, 1376, 160), (5, 256, 4, 704, 96)])
def test_decode_step_matches_cpu_restatement(cuda, built_libs, B, d, H, Fh, Smax):
    # one new token per sequence against a given FP8 KV cache: block output within the stated bar, the appended cache
    # rows equal to the restatement's up to isolated neighbouring codes (the RoPE runs in fp32 here, fp64 there)
    from goml_b200 import nn
    from oracle.decoder_block import decoder_block_decode_step
    cfg = f"blockdec{B}_{d}"
    hd = d // H
    blk, w, g1, g2, t = _make_block(cfg, d, H, Fh)
    k, sk, _ = O.quantize_f32(O.seeded_normal("k", (B, H, Smax, hd), config=cfg))
    v, sv, _ = O.quantize_f32(O.seeded_normal("v", (B, H, Smax, hd), config=cfg))
    positions = np.array([Smax - 1, 17, 64, 5, 90][:B], np.int32)
    x = O.seeded_normal("x", (B, d), config=cfg)
    cache = nn.FP8KVCache(B, H, Smax, hd)
    cache.k.copy_(torch.from_numpy(k)); cache.v.copy_(torch.from_numpy(v))
    cache.scales.copy_(torch.tensor([float(sk), float(sv)]))
    cache.lens.copy_(torch.from_numpy(positions))
    y = blk.decode_step(t(x), cache)
    torch.cuda.synchronize()
    blk.fa.DeviceStatus()
    ref, kr, vr = decoder_block_decode_step(x, positions, k, v, sk, sv, H, w["wqkv"], w["wo"], w["wgate_up"], w["wdown"], g1, g2)
    got = y.double().cpu().numpy()
    assert np.isfinite(got).all()
    maxabs, meanrel = O.error_stats(got, ref)
    assert maxabs <= 2e-2 and meanrel <= 1e-2, (maxabs, meanrel)
    maxabs_d, meanrel_d = O.error_stats(got - x, ref - x)
    assert maxabs_d <= 2e-2 and meanrel_d <= 5e-2, (maxabs_d, meanrel_d)
    assert np.array_equal(cache.lens.cpu().numpy(), positions + 1)
    for got_c, ref_c in ((cache.k.cpu().numpy(), kr), (cache.v.cpu().numpy(), vr)):
        differ = got_c != ref_c
        assert differ.mean() < 1e-4                        # only inside the appended rows, and rarely
        assert np.all(np.abs(got_c[differ].astype(int) - ref_c[differ].astype(int)) <= 1)
    blk.close()


def test_prompt_then_decode_equals_longer_prompt(cuda, built_libs):
    # the prompt fills the cache; decoding token S against it must reproduce row S of the block run over S + 1 tokens
    # (same arithmetic up to the per-tensor scales, which see one token more or less)
    from goml_b200 import nn
    B, S, d, H, Fh = 2, 128, 512, 4, 1376
    blk, w, g1, g2, t = _make_block("block-prefill-decode", d, H, Fh)
    x = O.seeded_normal("x", (B * (S + 1), d), config="block-prefill-decode").astype(np.float32).reshape(B, S + 1, d)
    full = blk(t(x.reshape(B * (S + 1), d)), B, S + 1).view(B, S + 1, d)
    cache = nn.FP8KVCache(B, H, S + 8, d // H)
    blk(t(np.ascontiguousarray(x[:, :S]).reshape(B * S, d)), B, S, cache)
    y = blk.decode_step(t(np.ascontiguousarray(x[:, S])), cache)
    torch.cuda.synchronize()
    blk.fa.DeviceStatus()
    assert cache.lens.tolist() == [S + 1] * B
    want = full[:, S].double().cpu().numpy()
    got = y.double().cpu().numpy()
    maxabs, meanrel = O.error_stats(got - x[:, S], want - x[:, S])
    assert maxabs <= 5e-2 and meanrel <= 1e-1, (maxabs, meanrel)          # what the block adds to the token's stream
    maxabs, meanrel = O.error_stats(got, want)
    assert maxabs <= 5e-2 and meanrel <= 1e-2, (maxabs, meanrel)
    blk.close()


def test_full_size_block_stage_by_stage(cuda, built_libs):
    """The block at its full configuration — d = 4096, 32 heads x 128, SwiGLU hidden 11008, 8 sequences x 2048 tokens
    (16384 rows) — run call by call exactly as FP8DecoderBlock.forward_fused issues it.  Every FP8 kernel stage is checked
    on the inputs the device itself produced (the same code bytes and scales are copied back): the GEMMs (tile pairs,
    SwiGLU / accumulate epilogues, TMA stores at N = 12288 / 22016 / 4096) on sampled token rows over all columns, the
    causal attention (BH = 256, S = 2048) on sampled (head, 32-row) blocks, the glue + quantise stages over the whole
    tensor.  The last stage's result is the block output."""
    import math
    from goml_b200 import block_glue as BG, fp8_gemm as G, nn
    from oracle import glue
    B, S, d, H, Fh = 8, 2048, 4096, 32, 11008
    T, hd = B * S, d // H
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(4)
    rn = lambda *shape, std=0.02: torch.randn(*shape, generator=g, device=dev) * std
    gam1, gam2 = 1.0 + 0.1 * rn(d, std=1.0), 1.0 + 0.1 * rn(d, std=1.0)
    blk = nn.FP8DecoderBlock(d, H, Fh, rn(3 * d, d), rn(d, d), rn(2 * Fh, d), rn(d, Fh), gam1, gam2)
    x = rn(T, d, std=1.0)
    u8 = lambda *shape: torch.empty(shape, dtype=torch.uint8, device=dev)
    sa = lambda n=2: torch.empty(n, dtype=torch.float32, device=dev)
    np_ = lambda t: t.detach().cpu().numpy()
    rows = np.unique(np.concatenate([[0, 127, 128, 2047, 2048, T - 129, T - 1], np.random.default_rng(3).integers(0, T, 25)]))
    rows_d = torch.from_numpy(rows).cuda()

    def sync():
        torch.cuda.synchronize()
        assert G.device_status() == 0
        blk.fa.DeviceStatus()

    def nearly_same_codes(got, want, frac=1e-4):
        key = lambda c: np.where(c.astype(np.int32) & 0x80, -(c.astype(np.int32) & 0x7f), c.astype(np.int32) & 0x7f)
        steps = np.abs(key(got) - key(want))
        assert steps.max() <= 1 and (steps != 0).mean() <= frac, (steps.max(), (steps != 0).mean())

    def close(got, ref, tol=(2e-2, 1e-2)):
        rms = float(np.sqrt(np.mean(ref ** 2)))
        maxabs, meanrel = O.error_stats(got / rms, ref / rms)
        assert maxabs <= tol[0] and meanrel <= tol[1], (maxabs, meanrel)

    # 1. RMSNorm + quantise (whole tensor)
    h = x.float().clone()
    rstd = torch.empty(T, dtype=torch.float32, device=dev)
    xq = nn.FP8Tensor(u8(T, d), sa())
    BG.RMSNormQuantize(h.data_ptr(), 0, 0, blk.norm1.data_ptr(), xq.codes.data_ptr(), xq.sa.data_ptr(), xq.sa.data_ptr() + 4,
                       rstd.data_ptr(), T, d, blk.eps)
    sync()
    codes, scale, amax, _, _ = glue.rmsnorm_quantize(np_(x), None, np_(blk.norm1), blk.eps)
    assert abs(xq.sa[0].item() - scale) <= 1e-6 * scale
    nearly_same_codes(np_(xq.codes), codes)

    # 2. QKV projection 16384 x 12288 x 4096, bf16 out (sampled rows, all columns)
    qkv = blk.qkv.forward_codes(xq, T)
    sync()
    alpha = float(np.float32(xq.sa[0].item()) * np.float32(blk.qkv.w.sa[0].item()))
    ref = O.gemm_f64(np_(xq.codes[rows_d]), np_(blk.qkv.w.codes), alpha)
    close(np_(qkv[rows_d].double()), ref, (2e-2, 3e-3))

    # 3. RoPE + head permute + quantise of Q, K, V (whole tensors, bit-exact)
    cos, sin = blk.rope_tables(S, dev)
    qc, kc, vc, s3 = u8(B * H, S, hd), u8(B * H, S, hd), u8(B * H, S, hd), sa(6)
    BG.RopeQuantizeQKV(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                       s3.data_ptr(), s3.data_ptr() + 12, B, S, H, hd)
    sync()
    want = glue.rope_quantize_qkv(np_(qkv.float()).reshape(T, 3, H, hd), np_(cos), np_(sin), B, S, H, hd)
    for got_c, (wc, wscale, _), i in zip((qc, kc, vc), want, range(3)):
        assert s3[i].item() == wscale and np.array_equal(np_(got_c), wc), i
    del want

    # 4. causal attention, BH = 256, S = 2048, D = 128 (sampled heads x row blocks)
    o = torch.zeros((B * H, S, hd), dtype=torch.float16, device=dev)
    blk.fa.ForwardEx(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), 0, B * H, S, hd, 1, 0, 1.0 / math.sqrt(hd), 1.0,
                     s3.data_ptr(), s3.data_ptr() + 4, s3.data_ptr() + 8)
    sync()
    sc = np_(s3)
    scale_qk = float(np.float32(1.0 / math.sqrt(hd)) * np.float32(sc[0]) * np.float32(sc[1]))
    for head, r0 in [(0, 0), (100, 1024 - 16), (255, 2048 - 32), (31, 96)]:
        qh, kh, vh = (np_(t[head:head + 1]) for t in (qc, kc, vc))
        ref, _ = O.attention_f64_rows(qh, kh, vh, r0, r0 + 32, 1, 0, scale_qk, float(sc[2]))
        maxabs, meanrel = O.error_stats(np_(o[head:head + 1, r0:r0 + 32].double()), ref)
        assert maxabs <= 2e-2 and meanrel <= 1e-2, (head, r0, maxabs, meanrel)

    # 5. head permute + quantise of the attention output (whole tensor, bit-exact)
    oq = nn.FP8Tensor(u8(T, d), sa())
    BG.PermuteQuantizeHeads(o.data_ptr(), oq.codes.data_ptr(), oq.sa.data_ptr(), oq.sa.data_ptr() + 4, B, S, H, hd)
    sync()
    wc, wscale, _ = glue.permute_quantize_heads(np_(o.float()), B, S, H, hd)
    assert oq.sa[0].item() == wscale and np.array_equal(np_(oq.codes), wc)

    # 6. O projection added into the fp32 stream in the GEMM epilogue (16384 x 4096 x 4096)
    h_before = np_(h[rows_d].double())
    blk.o.accumulate_into(oq, T, h)
    sync()
    alpha = float(np.float32(oq.sa[0].item()) * np.float32(blk.o.w.sa[0].item()))
    prod = O.gemm_f64(np_(oq.codes[rows_d]), np_(blk.o.w.codes), alpha)
    err = np.abs(np_(h[rows_d].double()) - (h_before + prod)).max()
    assert err <= 1e-5 * max(float(np.sqrt(np.mean(prod ** 2))), 1.0) * np.sqrt(d), err

    # 7. second RMSNorm + quantise (whole tensor)
    xq2 = nn.FP8Tensor(u8(T, d), sa())
    BG.RMSNormQuantize(h.data_ptr(), 0, 0, blk.norm2.data_ptr(), xq2.codes.data_ptr(), xq2.sa.data_ptr(), xq2.sa.data_ptr() + 4,
                       rstd.data_ptr(), T, d, blk.eps)
    sync()
    codes, scale, _, _, _ = glue.rmsnorm_quantize(np_(h), None, np_(blk.norm2), blk.eps)
    assert abs(xq2.sa[0].item() - scale) <= 1e-6 * scale
    nearly_same_codes(np_(xq2.codes), codes)

    # 8. gate/up projections with SwiGLU in the epilogue (16384 x 22016 x 4096 -> bf16 [16384, 11008] and max|H|)
    hq = nn.FP8Tensor(u8(T, Fh), sa())
    hb = torch.empty((T, Fh), dtype=torch.bfloat16, device=dev)
    G.FP8GEMMSwiGLU(T, Fh, d, xq2.codes.data_ptr(), blk.gate_up_interleaved.data_ptr(), hb.data_ptr(), 1.0, xq2.scale_ptr,
                    blk.gate_up.w.scale_ptr, hq.sa.data_ptr() + 4)
    sync()
    alpha = float(np.float32(xq2.sa[0].item()) * np.float32(blk.gate_up.w.sa[0].item()))
    gu = O.gemm_f64(np_(xq2.codes[rows_d]), np_(blk.gate_up.w.codes), alpha)
    gg, uu = gu[:, :Fh], gu[:, Fh:]
    ref = gg / (1.0 + np.exp(-gg)) * uu
    got = np_(hb[rows_d].double())
    assert np.all(np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-6 * np.abs(ref).max())
    assert hq.sa[1].item() == hb.float().abs().max().item()          # the epilogue's amax is the max of what it wrote

    # 9. quantiser pass over H (whole tensor, bit-exact against the restatement on the same bf16 values)
    BG.QuantizeBF16(hb.data_ptr(), hq.codes.data_ptr(), hq.sa.data_ptr(), hq.sa.data_ptr() + 4, T * Fh)
    sync()
    wc, wscale, _ = O.quantize_f32(np_(hb.float()))
    assert hq.sa[0].item() == wscale and np.array_equal(np_(hq.codes), wc)

    # 10. down projection added into the stream (16384 x 4096 x 11008): the block output
    h_before = np_(h[rows_d].double())
    blk.down.accumulate_into(hq, T, h)
    sync()
    alpha = float(np.float32(hq.sa[0].item()) * np.float32(blk.down.w.sa[0].item()))
    prod = O.gemm_f64(np_(hq.codes[rows_d]), np_(blk.down.w.codes), alpha)
    err = np.abs(np_(h[rows_d].double()) - (h_before + prod)).max()
    assert err <= 1e-5 * max(float(np.sqrt(np.mean(prod ** 2))), 1.0) * np.sqrt(Fh), err

    # the fused forward issues the same calls: same bits
    y = blk(x, B, S)
    sync()
    assert torch.equal(y, h)
    blk.close()
