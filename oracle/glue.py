"""CPU restatement (numpy) of the decoder block's row-local glue ops fused with the per-tensor e4m3
quantiser.  TEST INFRASTRUCTURE ONLY.

Arithmetic: internal/abjexam/battle_a_llm_f64ref.go:182-194 (rmsNorm, eps inside the square root),
:221-237 (half-split RoPE: pairs (i, i+hd/2), angle = pos * theta^(-2i/hd)), llama_hf_f64ref.go:160-178
(SwiGLU silu(gate) * up), evaluated in fp32 in the operation order the product documents, then the
quantiser of libs1/fp8_quantize_v2.cu:82-122 (scale = amax/448) through `oracle.quantize_f32`.
"""
import numpy as np

import oracle as O

f32 = np.float32


def bf16_values(a):
    """Round to bf16 and return the values as float32 (what a bf16 buffer holds)."""
    return O.round_bf16(np.asarray(a, np.float64)).astype(f32)


def rope_table(seq_len, head_dim, theta):
    half = head_dim // 2
    ang = np.arange(seq_len, dtype=np.float64)[:, None] * np.float64(theta) ** (-2.0 * np.arange(half, dtype=np.float64) / head_dim)
    return np.cos(ang).astype(f32), np.sin(ang).astype(f32)


def rmsnorm_quantize(x, residual, gamma, eps):
    """h = x (+ residual); y = (h * gamma) * rstd in fp32; returns (codes, scale, amax, h, y)."""
    h = np.asarray(x, f32)
    if residual is not None:
        h = h + np.asarray(residual, f32)
    ms = (h.astype(np.float64) ** 2).sum(-1).astype(f32) / f32(h.shape[-1])          # the product sums in fp32
    rstd = (1.0 / np.sqrt((ms + f32(eps)).astype(np.float64))).astype(f32)              # correctly rounded 1/sqrt
    y = (h * np.asarray(gamma, f32)[None, :]) * rstd[:, None]
    codes, scale, amax = O.quantize_f32(np.ascontiguousarray(y))
    return codes, scale, amax, h, y


def rope_quantize_qkv(qkv, cos, sin, B, S, H, hd):
    """qkv [B*S, 3, H, hd] float32 values -> (codes, scale) for Q, K, V as [B*H, S, hd]."""
    t = np.asarray(qkv, f32).reshape(B, S, 3, H, hd).transpose(2, 0, 3, 1, 4)  # [3, B, H, S, hd]
    half = hd // 2
    out = []
    for w in range(3):
        a = t[w]
        if w < 2:
            x0, x1 = a[..., :half], a[..., half:]
            a = np.concatenate([x0 * cos - x1 * sin, x0 * sin + x1 * cos], axis=-1)  # fp32: each product rounded, one add
        codes, scale, amax = O.quantize_f32(np.ascontiguousarray(a, f32).reshape(B * H, S, hd))
        out.append((codes, scale, amax))
    return out


def permute_quantize_heads(o, B, S, H, hd):
    """o [B*H, S, hd] float32 values of fp16 -> codes [B*S, H*hd]."""
    a = np.asarray(o, f32).reshape(B, H, S, hd).transpose(0, 2, 1, 3).reshape(B * S, H * hd)
    return O.quantize_f32(np.ascontiguousarray(a))


def swiglu_quantize(gu, F):
    """gu [rows, 2F] float32 values of bf16, gate columns first -> codes [rows, F]."""
    gu = np.asarray(gu, f32)
    g, u = gu[:, :F], gu[:, F:]
    e = np.exp(-g.astype(np.float64)).astype(f32)       # correctly rounded e^-g
    y = (g / (f32(1.0) + e)) * u
    codes, scale, amax = O.quantize_f32(np.ascontiguousarray(y))
    return codes, scale, amax, y


def decode_attention_f64(q, k_cache, v_cache, seq_lens, scale, v_descale=1.0):
    """One query token per sequence against a KV cache, grouped-query heads, fp64 (the arithmetic of
    internal/f64ref/attention.go:42-88 for a single query row: max-subtracted softmax over the visible keys,
    all-masked row -> zeros; LSE as defined in libs/fa_sm120/include/fa_sm120.h:100-102).
    q [B, Hq, D] e4m3 codes; k_cache, v_cache [B, Hkv, Smax, D] codes; seq_lens [B].  Returns (O [B, Hq, D], LSE [B, Hq])."""
    qf, kf, vf = (O.e4m3_decode(np.asarray(t, np.uint8)).astype(np.float64) for t in (q, k_cache, v_cache))
    B, Hq, D = qf.shape
    Hkv = kf.shape[1]
    group = Hq // Hkv
    out = np.zeros((B, Hq, D))
    lse = np.full((B, Hq), -np.inf)
    for b in range(B):
        n = int(seq_lens[b])
        if n <= 0:
            continue
        for h in range(Hq):
            kv = h // group
            s = kf[b, kv, :n] @ qf[b, h] * scale
            m = s.max()
            p = np.exp(s - m)
            out[b, h] = (p @ vf[b, kv, :n]) / p.sum() * v_descale
            lse[b, h] = m + np.log(p.sum())
    return out, lse


def quantize_fixed_scale(x, scale):
    """Codes of x for a tensor whose dequantisation scale is already fixed (an FP8 KV cache): the quantiser's second
    pass (libs1/fp8_quantize_v2.cu:100-121) with inv = 1/scale in fp32, clamp to +-448, round to nearest even."""
    inv = f32(1.0) / f32(scale)
    return O.e4m3_encode(np.clip(np.asarray(x, f32) * inv, f32(-448.0), f32(448.0)).astype(f32))


def decode_rope_append(qkv, cos, sin, positions, k_cache, v_cache, k_scale, v_scale, Hq, Hkv, hd):
    """The new token of every sequence: qkv [B, (Hq + 2*Hkv) * hd] float32 values of bf16 (query heads, key heads,
    value heads), half-split RoPE at positions[b] on Q and K (battle_a_llm_f64ref.go:221-237, evaluated in fp32: each
    product rounded, one add), Q quantised per tensor, K and V quantised with the cache's scales and written at
    position positions[b] of k_cache / v_cache [B, Hkv, Smax, hd] (KVCache.Append of
    runs/reports/F1_HF_INFERENCE_recon.md:186-196).  Sequences whose position is outside [0, min(Smax, rows of the
    RoPE table)) are inactive: zero Q codes, no append, length unchanged (0 for a negative position, else min(position, Smax)).
    Returns (q_codes [B, Hq, hd], q_scale, q_amax, k_cache', v_cache', seq_lens)."""
    qkv = np.asarray(qkv, f32)
    B = qkv.shape[0]
    Smax = k_cache.shape[2]
    half = hd // 2
    rows = qkv.reshape(B, Hq + 2 * Hkv, hd)
    kc, vc = k_cache.copy(), v_cache.copy()
    qv = np.zeros((B, Hq, hd), f32)
    active = np.zeros(B, bool)
    seq_lens = np.zeros(B, np.int32)

    def rope(a, pos):
        x0, x1 = a[..., :half], a[..., half:]
        c, s = cos[pos], sin[pos]
        return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1).astype(f32)

    for b in range(B):
        pos = int(positions[b])
        if not (0 <= pos < min(Smax, cos.shape[0])):
            seq_lens[b] = 0 if pos < 0 else min(pos, Smax)      # inactive: the length stays as it is
            continue
        active[b] = True
        seq_lens[b] = pos + 1
        qv[b] = rope(rows[b, :Hq], pos)
        kc[b, :, pos] = quantize_fixed_scale(rope(rows[b, Hq:Hq + Hkv], pos), k_scale)
        vc[b, :, pos] = quantize_fixed_scale(rows[b, Hq + Hkv:], v_scale)
    amax = f32(np.abs(qv[active]).max()) if active.any() else f32(0.0)
    scale = f32(amax / f32(448.0)) if amax > 1e-12 else f32(1.0)
    q_codes = quantize_fixed_scale(qv, scale)
    q_codes[~active] = 0
    return q_codes, scale, amax, kc, vc, seq_lens
