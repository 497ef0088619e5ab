"""Host-side logic that needs no GPU: the weight layout of the SwiGLU GEMM, and the consistency of the CPU
restatements with each other (decode step = last causal row of the prefill restatement; glue restatements against
the fp64 block restatement's intermediates)."""
import math

import numpy as np

import oracle as O
from oracle import glue
from oracle.decoder_block import decoder_block


def test_interleave_gate_up_layout():
    from goml_b200.fp8_gemm import interleave_gate_up
    F, K = 300, 5
    w = (np.arange(2 * F * K) % 251).astype(np.uint8).reshape(2 * F, K)
    wi = interleave_gate_up(w, F)
    Fp = 320
    assert wi.shape == (2 * Fp, K)
    for t in range(Fp // 32):
        for r in range(32):
            col = 32 * t + r
            want_g = w[col] if col < F else np.zeros(K, np.uint8)
            want_u = w[F + col] if col < F else np.zeros(K, np.uint8)
            assert np.array_equal(wi[64 * t + r], want_g) and np.array_equal(wi[64 * t + 32 + r], want_u)
    import torch
    assert np.array_equal(interleave_gate_up(torch.from_numpy(w), F).numpy(), wi)      # the torch path builds the same layout


def test_decode_restatement_is_the_last_causal_row_of_the_prefill_restatement():
    B, Hkv, S, D, group = 2, 2, 70, 64, 2
    q_full, sq, _ = O.quantize_f32(O.seeded_normal("q", (B * Hkv * group, S, D), config="dec-cpu"))
    k, sk, _ = O.quantize_f32(O.seeded_normal("k", (B * Hkv, S, D), config="dec-cpu"))
    v, sv, _ = O.quantize_f32(O.seeded_normal("v", (B * Hkv, S, D), config="dec-cpu"))
    scale = float(sq) * float(sk) / math.sqrt(D)
    # prefill restatement per query head on its kv head's cache
    kk = np.repeat(k.reshape(B, Hkv, S, D), group, axis=1).reshape(B * Hkv * group, S, D)
    vv = np.repeat(v.reshape(B, Hkv, S, D), group, axis=1).reshape(B * Hkv * group, S, D)
    o_pre, l_pre = O.attention_f64(q_full, kk, vv, 1, 0, scale, float(sv))
    q_last = q_full[:, S - 1].reshape(B, Hkv * group, D)
    o_dec, l_dec = glue.decode_attention_f64(q_last, k.reshape(B, Hkv, S, D), v.reshape(B, Hkv, S, D), [S] * B, scale, float(sv))
    assert np.abs(o_dec.reshape(-1, D) - o_pre[:, S - 1]).max() <= 1e-12
    assert np.abs(l_dec.reshape(-1) - l_pre[:, S - 1]).max() <= 1e-12


def test_glue_restatements_agree_with_the_block_restatement():
    B, S, d, H, Fh = 1, 32, 128, 2, 256
    cfg = "glue-cpu"
    w = {n: O.seeded_normal(n, shp, std=0.05, config=cfg) for n, shp in
         dict(wqkv=(3 * d, d), wo=(d, d), wgate_up=(2 * Fh, d), wdown=(d, Fh)).items()}
    g = 1.0 + 0.1 * O.seeded_normal("g", (d,), config=cfg)
    x = O.seeded_normal("x", (B * S, d), config=cfg)
    inter = {}
    decoder_block(x, B, S, H, w["wqkv"], w["wo"], w["wgate_up"], w["wdown"], g, g, intermediates=inter)
    # RMSNorm + quantise: the fp32 restatement quantises what the fp64 block restatement normalises
    codes, scale, amax, _, y = glue.rmsnorm_quantize(x.astype(np.float32), None, g.astype(np.float32), 1e-5)
    assert np.abs(y - inter["xn1"]).max() <= 1e-5
    want_codes, want_scale, _ = O.quantize_f32(inter["xn1"].astype(np.float32))
    assert abs(scale - want_scale) <= 1e-6 * want_scale and (codes != want_codes).mean() <= 1e-3
    # SwiGLU + quantise on the block's bf16 gate/up projection
    codes, scale, amax, h = glue.swiglu_quantize(glue.bf16_values(inter["gu"]), Fh)
    assert np.abs(h - inter["h"]).max() <= 1e-5 * max(1.0, np.abs(inter["h"]).max())
    # RoPE tables: fp64 angles rounded once
    c, s = glue.rope_table(S, d // H, 10000.0)
    assert c.dtype == np.float32 and np.abs(c.astype(np.float64) ** 2 + s.astype(np.float64) ** 2 - 1).max() <= 3e-7


def test_decode_append_restatement_properties():
    # the appended K row decodes to RoPE(k) within one e4m3 step of the cache scale, positions outside the cache are
    # inactive, nothing but the appended rows changes, and position 0 (angle 0) leaves Q and K un-rotated
    B, Hq, Hkv, S, hd = 4, 4, 2, 32, 64
    cos, sin = glue.rope_table(S, hd, 10000.0)
    qkv = O.round_bf16(O.seeded_normal("qkv", (B, (Hq + 2 * Hkv) * hd), config="append-cpu")).astype(np.float32)
    k, sk, _ = O.quantize_f32(O.seeded_normal("k", (B, Hkv, S, hd), config="append-cpu"))
    v, sv, _ = O.quantize_f32(O.seeded_normal("v", (B, Hkv, S, hd), config="append-cpu"))
    positions = [0, 7, S, -1]
    qc, qs, qa, kc, vc, lens = glue.decode_rope_append(qkv, cos, sin, positions, k, v, sk, sv, Hq, Hkv, hd)
    assert list(lens) == [1, 8, S, 0]
    assert np.all(qc[2:] == 0) and np.array_equal(kc[2:], k[2:]) and np.array_equal(vc[2:], v[2:])
    changed = np.zeros_like(k, bool)
    changed[0, :, 0] = changed[1, :, 7] = True
    assert np.array_equal(kc[~changed], k[~changed]) and np.array_equal(vc[~changed], v[~changed])
    rows = qkv.reshape(B, Hq + 2 * Hkv, hd)
    # position 0: cos = 1, sin = 0 -> codes of the un-rotated rows
    assert np.array_equal(kc[0, :, 0], glue.quantize_fixed_scale(rows[0, Hq:Hq + Hkv], sk))
    assert np.array_equal(vc[1, :, 7], glue.quantize_fixed_scale(rows[1, Hq + Hkv:], sv))
    assert qs == np.float32(qa / np.float32(448.0))
    # rotation preserves the norm of every (i, i + hd/2) pair
    kd = O.e4m3_decode(kc[1, :, 7]).astype(np.float64) * float(sk)
    kin = rows[1, Hq:Hq + Hkv].astype(np.float64)
    n_out = kd[:, :hd // 2] ** 2 + kd[:, hd // 2:] ** 2
    n_in = kin[:, :hd // 2] ** 2 + kin[:, hd // 2:] ** 2
    assert np.abs(np.sqrt(n_out) - np.sqrt(n_in)).max() <= 0.07 * np.abs(kin).max()    # one e4m3 step (2^-4 relative)


def test_fixed_scale_quantiser_saturates():
    codes = glue.quantize_fixed_scale(np.array([1e6, -1e6, 0.0, 448.0, 0.5], np.float32), 1.0)
    assert list(codes) == [0x7E, 0xFE, 0x00, 0x7E, 0x30]
