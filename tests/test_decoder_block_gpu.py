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
