"""CPU restatement (numpy, fp64) of one Llama-style decoder block with the FP8 quantisation points
of the product chain.  TEST INFRASTRUCTURE ONLY.

Arithmetic follows internal/abjexam/llama_hf_f64ref.go:94-178 (pre-norm block, y = x W^T with W [out,in],
[S,H,hd] -> [H,S,hd], causal attention, SwiGLU silu(gate)*up, residuals) with the primitives of
internal/abjexam/battle_a_llm_f64ref.go:182-194 (rmsNorm: eps inside the square root) and :221-237
(half-split RoPE: pairs (i, i+hd/2), angle = pos * theta^(-2i/hd)).  Every GEMM operand and Q/K/V are
quantised per tensor to e4m3 (scale = amax/448) exactly where the product quantises; GEMM results are
rounded to bf16 and the attention output to fp16, as the libraries return them.
"""
import math

import numpy as np

import oracle as O


def _linear(x, w, round_out=True):
    """bf16( sx*sw * codes(x) . codes(w)^T ), fp64 accumulation; un-rounded when the product adds the result
    into the fp32 residual stream inside the GEMM epilogue."""
    xq, sx, _ = O.quantize_f32(x.astype(np.float32))
    wq, sw, _ = O.quantize_f32(w.astype(np.float32))
    alpha = float(np.float32(sx) * np.float32(sw))  # the kernel multiplies the fp32 scales
    y = O.gemm_f64(xq, wq, alpha)
    return O.round_bf16(y).astype(np.float64) if round_out else y


def _rms_norm(x, gamma, eps):
    return gamma * x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def _rope(x, theta):  # x [B, H, S, hd]
    hd, S = x.shape[-1], x.shape[-2]
    half = hd // 2
    freq = theta ** (-2.0 * np.arange(half) / hd)
    ang = np.arange(S)[:, None] * freq[None, :]
    c, s = np.cos(ang), np.sin(ang)
    x0, x1 = x[..., :half], x[..., half:]
    return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1)


def decoder_block(x, B, S, H, wqkv, wo, wgate_up, wdown, norm1, norm2, eps=1e-5, theta=10000.0, intermediates=None,
                  residual_in_epilogue=False, swiglu_in_epilogue=False):
    """Returns the block output [B*S, d] (fp64).  When `intermediates` is a dict it receives the input of
    every quantised stage and that stage's output, so each product stage can be checked on identical inputs.
    `residual_in_epilogue`: the O and down projections are added to the stream un-rounded (fp32 accumulators),
    as the product's fused path does; otherwise they are rounded to bf16 first.
    `swiglu_in_epilogue`: silu(gate) * up is taken on the un-rounded gate/up projections and rounded to bf16 once."""
    x = x.astype(np.float64)
    d = x.shape[1]
    hd = d // H
    Fh = wdown.shape[1]
    keep = intermediates if intermediates is not None else {}
    keep["xn1"] = _rms_norm(x, norm1, eps)
    keep["qkv"] = _linear(keep["xn1"], wqkv)
    qkv = keep["qkv"].reshape(B, S, 3, H, hd).transpose(2, 0, 3, 1, 4)
    q, k, v = _rope(qkv[0], theta), _rope(qkv[1], theta), qkv[2]
    (qq, sq, _), (kq, sk, _), (vq, sv, _) = [O.quantize_f32(np.ascontiguousarray(t, np.float32).reshape(B * H, S, hd)) for t in (q, k, v)]
    scale = float(np.float32(1.0 / math.sqrt(hd)) * np.float32(sq) * np.float32(sk))
    o, _ = O.attention_f64(qq, kq, vq, 1, 0, scale, float(sv))
    keep["attn"] = O.round_fp16(o).astype(np.float64).reshape(B, H, S, hd).transpose(0, 2, 1, 3).reshape(B * S, d)
    keep["ao"] = _linear(keep["attn"], wo, round_out=not residual_in_epilogue)
    x = x + keep["ao"]
    keep["x_mid"] = x
    keep["xn2"] = _rms_norm(x, norm2, eps)
    keep["gu"] = _linear(keep["xn2"], wgate_up, round_out=not swiglu_in_epilogue)
    g, u = keep["gu"][:, :Fh], keep["gu"][:, Fh:]
    keep["h"] = g / (1.0 + np.exp(-g)) * u
    if swiglu_in_epilogue:
        keep["h"] = O.round_bf16(keep["h"]).astype(np.float64)
    keep["ffn"] = _linear(keep["h"], wdown, round_out=not residual_in_epilogue)
    return x + keep["ffn"]


def decoder_block_decode_step(x, positions, k_cache, v_cache, k_scale, v_scale, H, wqkv, wo, wgate_up, wdown, norm1, norm2,
                              eps=1e-5, theta=10000.0, intermediates=None):
    """One new token per sequence through the same block (fp64, the product's quantisation points): x [B, d] is the
    token's residual stream, k_cache / v_cache [B, H, Smax, hd] e4m3 codes with dequantisation scales k_scale / v_scale,
    positions[b] the number of keys already cached.  The token's K (after RoPE at its position) and V are quantised
    with the cache's scales and written at positions[b] (KVCache.Append of runs/reports/F1_HF_INFERENCE_recon.md:186-196),
    then the token attends to keys [0, positions[b]] (the single-row case of the causal attention of
    internal/abjexam/llama_hf_f64ref.go:94-178).  The residual adds and SwiGLU use un-rounded projections, as the fused
    product path does.  Returns (y [B, d], k_cache', v_cache')."""
    from oracle import glue
    x = x.astype(np.float64)
    B, d = x.shape
    hd = d // H
    Fh = wdown.shape[1]
    half = hd // 2
    keep = intermediates if intermediates is not None else {}
    keep["xn1"] = _rms_norm(x, norm1, eps)
    keep["qkv"] = _linear(keep["xn1"], wqkv)
    rows = keep["qkv"].reshape(B, 3, H, hd)
    freq = theta ** (-2.0 * np.arange(half) / hd)
    ang = np.asarray(positions, np.float64)[:, None, None] * freq[None, None, :]
    c, s = np.cos(ang), np.sin(ang)

    def rope(a):
        x0, x1 = a[..., :half], a[..., half:]
        return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1)

    q, k, v = rope(rows[:, 0]), rope(rows[:, 1]), rows[:, 2]
    qq, sq, _ = O.quantize_f32(np.ascontiguousarray(q, np.float32))
    kc, vc = k_cache.copy(), v_cache.copy()
    for b in range(B):
        kc[b, :, int(positions[b])] = glue.quantize_fixed_scale(k[b].astype(np.float32), k_scale)
        vc[b, :, int(positions[b])] = glue.quantize_fixed_scale(v[b].astype(np.float32), v_scale)
    scale = float(np.float32(1.0 / math.sqrt(hd)) * np.float32(sq) * np.float32(k_scale))
    o, _ = glue.decode_attention_f64(qq, kc, vc, np.asarray(positions) + 1, scale, float(v_scale))
    keep["attn"] = O.round_fp16(o).astype(np.float64).reshape(B, d)
    keep["ao"] = _linear(keep["attn"], wo, round_out=False)
    x = x + keep["ao"]
    keep["xn2"] = _rms_norm(x, norm2, eps)
    keep["gu"] = _linear(keep["xn2"], wgate_up, round_out=False)
    g, u = keep["gu"][:, :Fh], keep["gu"][:, Fh:]
    keep["h"] = O.round_bf16(g / (1.0 + np.exp(-g)) * u).astype(np.float64)
    keep["ffn"] = _linear(keep["h"], wdown, round_out=False)
    return x + keep["ffn"], kc, vc
