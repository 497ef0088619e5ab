"""FP8 dispatch of goml's nn call sites for one Llama-style decoder block (prefill).

goml's `nn.Linear.Forward` (nn/linear.go:53-74), `nn.FeedForward.forwardSwiGLU`
(nn/feedforward.go:54-79: W2(silu(W1 x) * W3 x)) and `nn.MultiHeadAttention.Forward`
(nn/attention.go:60-160) run in F32 today.  Here every projection goes through the FP8
GEMM library, the attention through the FP8 attention library and every quantisation
through the quantiser library — scales stay on the device between them (no host round
trip).  The row-local glue (RMSNorm with eps inside the square root, half-split RoPE, SiLU
gate, residual adds, layout permutes: the arithmetic of
internal/abjexam/llama_hf_f64ref.go:126-178 and battle_a_llm_f64ref.go:182-237) runs
through libfp8block.so, each op fused with the quantiser of the next GEMM / attention
operand (`fused=True`, the default), or as plain fp32 torch ops followed by separate
quantiser calls (`fused=False`, kept as the unfused comparison).

torch tensors are used as device buffers; all heavy kernels are reached through the C ABI.
"""
from __future__ import annotations

import math

import torch

from . import block_glue as BG, fa_forward as F, fp8_gemm as G, quantize as Q


class FP8Tensor:
    """e4m3 codes + a one-float device scale (and the amax word the quantiser writes)."""

    def __init__(self, codes: torch.Tensor, scale_amax: torch.Tensor):
        self.codes = codes
        self.sa = scale_amax  # [scale, amax] fp32 on the device

    @property
    def scale_ptr(self) -> int:
        return self.sa.data_ptr()


def quantize(x: torch.Tensor, unit: bool = False) -> FP8Tensor:
    """Per-tensor FP32 -> e4m3 through libfp8quant (scale = amax/448, or amax when unit)."""
    x = x.contiguous()
    assert x.dtype == torch.float32 and x.is_cuda
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    sa = torch.zeros(2, dtype=torch.float32, device=x.device)
    fn = Q.QuantizeF32ToF8E4M3Unit if unit else Q.QuantizeF32ToF8E4M3
    fn(x.data_ptr(), codes.data_ptr(), sa.data_ptr(), sa.data_ptr() + 4, x.numel(), torch.cuda.current_stream().cuda_stream)
    return FP8Tensor(codes, sa)


class FP8Linear:
    """y = x W^T with W [out, in] (the layout of nn/linear.go:14), both operands e4m3, bf16 result."""

    def __init__(self, weight: torch.Tensor):
        self.out_features, self.in_features = weight.shape
        self.w = quantize(weight.float())

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        M = x.numel() // self.in_features
        return self.forward_codes(quantize(x.reshape(M, self.in_features).float()), M)

    def accumulate_into(self, xq: FP8Tensor, M: int, x: torch.Tensor) -> None:
        """x (fp32 [M, out]) += this layer's output, added in the GEMM epilogue (no 16-bit intermediate)."""
        assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (M, self.out_features)
        G.FP8GEMMAccumulateF32(M, self.out_features, self.in_features, xq.codes.data_ptr(), self.w.codes.data_ptr(), x.data_ptr(),
                               1.0, xq.scale_ptr, self.w.scale_ptr, torch.cuda.current_stream().cuda_stream)

    def forward_codes(self, xq: FP8Tensor, M: int) -> torch.Tensor:
        """The GEMM alone, on an activation that is already e4m3 codes + device scale."""
        y = torch.empty((M, self.out_features), dtype=torch.bfloat16, device=xq.codes.device)
        G.FP8GEMMScaled(M, self.out_features, self.in_features, xq.codes.data_ptr(), self.w.codes.data_ptr(), y.data_ptr(),
                        1.0, xq.scale_ptr, self.w.scale_ptr, G.OutBF16, torch.cuda.current_stream().cuda_stream)
        return y


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    return gamma * x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rope_half_split(x: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B, H, S, hd]: pairs (i, i + hd/2), angle = pos * theta^(-2i/hd)."""
    hd, S = x.shape[-1], x.shape[-2]
    half = hd // 2
    freq = theta ** (-2.0 * torch.arange(half, device=x.device, dtype=torch.float64) / hd)
    ang = torch.arange(S, device=x.device, dtype=torch.float64)[:, None] * freq[None, :]
    c, s = ang.cos().float(), ang.sin().float()
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


class FP8KVCache:
    """One layer's FP8 KV cache: K and V codes [batch, heads, s_max, hd] with one dequantisation scale each, fixed
    when the prompt is written, and the per-sequence lengths on the device.  The structure of the KVCache sketched in
    goml's runs/reports/F1_HF_INFERENCE_recon.md:186-196 (Append at position tCur, K()/V() views), holding e4m3 codes
    instead of fp32 and S_max allocated up front."""

    def __init__(self, batch: int, heads: int, s_max: int, hd: int, device="cuda"):
        self.B, self.H, self.s_max, self.hd = batch, heads, s_max, hd
        self.k = torch.zeros((batch, heads, s_max, hd), dtype=torch.uint8, device=device)
        self.v = torch.zeros_like(self.k)
        self.scales = torch.ones(2, dtype=torch.float32, device=device)      # k_scale, v_scale
        self.lens = torch.zeros(batch, dtype=torch.int32, device=device)     # keys cached per sequence
        self._lens_next = torch.zeros_like(self.lens)

    def fill(self, k_codes, v_codes, scales, S: int) -> None:
        """Prompt phase: K/V codes [batch*heads, S, hd] as the prefill quantiser wrote them, and their two scales."""
        self.k[:, :, :S].copy_(k_codes.view(self.B, self.H, S, self.hd))
        self.v[:, :, :S].copy_(v_codes.view(self.B, self.H, S, self.hd))
        self.scales.copy_(scales)
        self.lens.fill_(S)


class FP8DecoderBlock:
    """Llama-style block: RMSNorm -> QKV -> RoPE -> causal FP8 attention -> O -> residual -> RMSNorm -> SwiGLU -> residual."""

    def __init__(self, d_model, n_heads, ffn_hidden, wqkv, wo, wgate_up, wdown, norm1, norm2, eps=1e-5, theta=10000.0, fused=True):
        self.fused = fused
        self._rope = {}   # seq_len -> (cos, sin) device tables
        self.d, self.H, self.F = d_model, n_heads, ffn_hidden
        self.hd = d_model // n_heads
        assert self.hd in (64, 128)
        self.qkv, self.o = FP8Linear(wqkv), FP8Linear(wo)
        self.gate_up, self.down = FP8Linear(wgate_up), FP8Linear(wdown)
        # the same gate/up codes in the layout the SwiGLU GEMM epilogue reads (gate and up rows of a column block adjacent)
        self.gate_up_interleaved = G.interleave_gate_up(self.gate_up.w.codes, ffn_hidden)
        self.norm1, self.norm2 = norm1.float(), norm2.float()
        self.eps, self.theta = eps, theta
        self.fa = F.FACreate()

    def attention(self, xn: torch.Tensor, B: int, S: int) -> torch.Tensor:
        H, hd = self.H, self.hd
        qkv = self.qkv(xn).float().view(B, S, 3, H, hd).permute(2, 0, 3, 1, 4)  # [3, B, H, S, hd]
        q = rope_half_split(qkv[0], self.theta)
        k = rope_half_split(qkv[1], self.theta)
        qq, kq, vq = quantize(q), quantize(k), quantize(qkv[2])
        o = torch.empty((B * H, S, hd), dtype=torch.float16, device=xn.device)
        self.fa.ForwardEx(qq.codes.data_ptr(), kq.codes.data_ptr(), vq.codes.data_ptr(), o.data_ptr(), 0, B * H, S, hd, 1, 0,
                          1.0 / math.sqrt(hd), 1.0, qq.scale_ptr, kq.scale_ptr, vq.scale_ptr, torch.cuda.current_stream().cuda_stream)
        return o.view(B, H, S, hd).permute(0, 2, 1, 3).reshape(B * S, H * hd)

    def rope_tables(self, S: int, dev) -> tuple[torch.Tensor, torch.Tensor]:
        if S not in self._rope:
            cos = torch.empty((S, self.hd // 2), dtype=torch.float32, device=dev)
            sin = torch.empty_like(cos)
            BG.RopeTable(cos.data_ptr(), sin.data_ptr(), S, self.hd, self.theta, torch.cuda.current_stream().cuda_stream)
            self._rope[S] = (cos, sin)
        return self._rope[S]

    def forward_fused(self, x: torch.Tensor, B: int, S: int, cache: "FP8KVCache | None" = None) -> torch.Tensor:
        """The block with every glue op fused with the quantiser of its consumer and both residual adds done in
        the GEMM epilogues, SwiGLU in the gate/up GEMM's epilogue: 9 library calls, no torch math.
        With `cache`, the K and V codes of the prompt and their scales are also stored there for decode_step."""
        dev, T, d, H, hd, Fh = x.device, B * S, self.d, self.H, self.hd, self.F
        sh = torch.cuda.current_stream().cuda_stream
        u8 = lambda *shape: torch.empty(shape, dtype=torch.uint8, device=dev)
        sa = lambda n=2: torch.empty(n, dtype=torch.float32, device=dev)   # scale and amax words: every entry point clears its own amax
        h = x.float().clone()                                   # residual stream, updated in place
        rstd = torch.empty(T, dtype=torch.float32, device=dev)
        cos, sin = self.rope_tables(S, dev)
        # attention half
        xq = FP8Tensor(u8(T, d), sa())
        BG.RMSNormQuantize(h.data_ptr(), 0, 0, self.norm1.data_ptr(), xq.codes.data_ptr(), xq.sa.data_ptr(), xq.sa.data_ptr() + 4,
                           rstd.data_ptr(), T, d, self.eps, sh)
        qkv = self.qkv.forward_codes(xq, T)                      # [T, 3, H, hd] bf16
        qc, kc, vc, s3 = u8(B * H, S, hd), u8(B * H, S, hd), u8(B * H, S, hd), sa(6)   # scales[3], amaxes[3]
        BG.RopeQuantizeQKV(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                           s3.data_ptr(), s3.data_ptr() + 12, B, S, H, hd, sh)
        if cache is not None:
            cache.fill(kc, vc, s3[1:3], S)
        o = torch.empty((B * H, S, hd), dtype=torch.float16, device=dev)
        self.fa.ForwardEx(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), 0, B * H, S, hd, 1, 0, 1.0 / math.sqrt(hd), 1.0,
                          s3.data_ptr(), s3.data_ptr() + 4, s3.data_ptr() + 8, sh)
        oq = FP8Tensor(u8(T, d), sa())
        BG.PermuteQuantizeHeads(o.data_ptr(), oq.codes.data_ptr(), oq.sa.data_ptr(), oq.sa.data_ptr() + 4, B, S, H, hd, sh)
        self.o.accumulate_into(oq, T, h)                         # h += attention projection, in the GEMM epilogue
        return self._feed_forward(h, T)

    def decode_step(self, x: torch.Tensor, cache: FP8KVCache) -> torch.Tensor:
        """One new token per sequence: x [batch, d] fp32 -> [batch, d] fp32, the token's K and V appended to `cache` at
        position cache.lens[b] (quantised with the cache's scales) and cache.lens advanced.  Ten library calls:
        RMSNorm+quantise -> QKV GEMM -> RoPE+quantise+append -> decode attention -> quantise -> O GEMM (residual in the
        epilogue) -> the feed-forward half of forward_fused."""
        dev, B, d, H, hd = x.device, x.shape[0], self.d, self.H, self.hd
        assert (B, H, hd) == (cache.B, cache.H, cache.hd)
        sh = torch.cuda.current_stream().cuda_stream
        u8 = lambda *shape: torch.empty(shape, dtype=torch.uint8, device=dev)
        sa = lambda n=2: torch.empty(n, dtype=torch.float32, device=dev)
        h = x.float().clone()
        rstd = torch.empty(B, dtype=torch.float32, device=dev)
        cos, sin = self.rope_tables(cache.s_max, dev)
        xq = FP8Tensor(u8(B, d), sa())
        BG.RMSNormQuantize(h.data_ptr(), 0, 0, self.norm1.data_ptr(), xq.codes.data_ptr(), xq.sa.data_ptr(), xq.sa.data_ptr() + 4,
                           rstd.data_ptr(), B, d, self.eps, sh)
        qkv = self.qkv.forward_codes(xq, B)                      # [B, (H + 2H) * hd] bf16: Q heads, K heads, V heads
        qc, qs = u8(B, H, hd), sa()
        BG.DecodeRopeAppend(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), cache.lens.data_ptr(), qc.data_ptr(), qs.data_ptr(),
                            qs.data_ptr() + 4, cache.k.data_ptr(), cache.v.data_ptr(), cache.scales.data_ptr(), cache.scales.data_ptr() + 4,
                            B, H, H, hd, cache.s_max, cache.s_max, seq_lens_out=cache._lens_next.data_ptr(), stream=sh)
        cache.lens.copy_(cache._lens_next)    # a device copy, not a pointer swap: the step can be replayed from a CUDA graph
        o = torch.empty((B, H, hd), dtype=torch.float16, device=dev)
        self.fa.Decode(qc.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), o.data_ptr(), 0, cache.lens.data_ptr(), B, H, H, hd,
                       cache.s_max, 0, 1.0 / math.sqrt(hd), 1.0, qs.data_ptr(), cache.scales.data_ptr(), cache.scales.data_ptr() + 4, sh)
        oq = FP8Tensor(u8(B, d), sa())
        BG.PermuteQuantizeHeads(o.data_ptr(), oq.codes.data_ptr(), oq.sa.data_ptr(), oq.sa.data_ptr() + 4, B, 1, H, hd, sh)
        self.o.accumulate_into(oq, B, h)
        return self._feed_forward(h, B)

    def _feed_forward(self, h: torch.Tensor, T: int) -> torch.Tensor:
        """h [T, d] fp32 += W_down(silu(W_gate n) * W_up n), n = RMSNorm(h): in place, three GEMM-library calls."""
        dev, d, Fh = h.device, self.d, self.F
        sh = torch.cuda.current_stream().cuda_stream
        u8 = lambda *shape: torch.empty(shape, dtype=torch.uint8, device=dev)
        sa = lambda n=2: torch.empty(n, dtype=torch.float32, device=dev)
        rstd = torch.empty(T, dtype=torch.float32, device=dev)
        xq2 = FP8Tensor(u8(T, d), sa())
        BG.RMSNormQuantize(h.data_ptr(), 0, 0, self.norm2.data_ptr(), xq2.codes.data_ptr(), xq2.sa.data_ptr(),
                           xq2.sa.data_ptr() + 4, rstd.data_ptr(), T, d, self.eps, sh)
        hq = FP8Tensor(u8(T, Fh), sa())
        hb = torch.empty((T, Fh), dtype=torch.bfloat16, device=dev)
        # gate/up projections with silu(gate) * up and max|.| in the GEMM epilogue, then one quantiser pass
        G.FP8GEMMSwiGLU(T, Fh, d, xq2.codes.data_ptr(), self.gate_up_interleaved.data_ptr(), hb.data_ptr(), 1.0, xq2.scale_ptr,
                        self.gate_up.w.scale_ptr, hq.sa.data_ptr() + 4, sh)
        BG.QuantizeBF16(hb.data_ptr(), hq.codes.data_ptr(), hq.sa.data_ptr(), hq.sa.data_ptr() + 4, T * Fh, sh)
        self.down.accumulate_into(hq, T, h)                      # h += feed-forward output
        return h

    def __call__(self, x: torch.Tensor, B: int, S: int, cache: "FP8KVCache | None" = None) -> torch.Tensor:
        """x [B*S, d] fp32 -> [B*S, d] fp32."""
        assert cache is None or self.fused, "the KV cache is written by the fused path"
        if self.fused:
            return self.forward_fused(x, B, S, cache)
        x = x.float()
        x = x + self.o(self.attention(rms_norm(x, self.norm1, self.eps), B, S)).float()
        gu = self.gate_up(rms_norm(x, self.norm2, self.eps)).float()
        g, u = gu[:, : self.F], gu[:, self.F:]
        x = x + self.down(torch.nn.functional.silu(g) * u).float()
        return x

    def close(self):
        self.fa.Destroy()


def _main():
    """Times the full-size block config: d_model 4096, 32 heads x 128, SwiGLU hidden 11008, B=8 x S=2048
    tokens, random-init weights N(0, 0.02), embeddings N(0, 1) — the whole block and its FP8 kernels alone."""
    import os
    import sys
    B, S, d, H, Fh = 8, 2048, 4096, 32, 11008
    if len(sys.argv) > 1:
        B = int(sys.argv[1])
    # Under torchrun the block is sharded by rows on sequence boundaries (the M-tile partition of the GEMMs and the
    # batch*head partition of the attention coincide there): weights replicated, no collective on the data path;
    # torch.distributed is used for the barrier and the max-over-ranks of the timing only.
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        from .multi_gpu import shard_rows
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        lo, hi = shard_rows(B * S, world, rank, tile=S)      # whole sequences per rank
        B_global, B = B, (hi - lo) // S
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(4)
    rn = lambda *shape, std=0.02: torch.randn(*shape, generator=g, device=dev) * std
    blk = FP8DecoderBlock(d, H, Fh, rn(3 * d, d), rn(d, d), rn(2 * Fh, d), rn(d, Fh), torch.ones(d, device=dev), torch.ones(d, device=dev))
    x = rn(B * S, d, std=1.0)

    def timed(fn, iters=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    if world > 1:
        dist.barrier()
        t = torch.tensor([timed(lambda: blk(x, B, S), iters=10)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            fl = 2.0 * B_global * S * d * (3 * d + d + 3 * Fh) + 2.0 * B_global * H * S * S * (d // H)
            print(f"block B={B_global} S={S} d={d} H={H} F={Fh} over {world} GPUs ({B} sequences per GPU, no collective): "
                  f"{t.item():.3f} ms (max over ranks) = {fl / t.item() / 1e9:.0f} TFLOPS whole job")
        blk.close()
        dist.destroy_process_group()
        return
    total = timed(lambda: blk(x, B, S))
    blk.fused = False
    total_unfused = timed(lambda: blk(x, B, S))
    blk.fused = True
    M = B * S
    # kernels alone, on pre-quantised operands
    xq = quantize(x)
    sh = torch.cuda.current_stream().cuda_stream

    def gemm(lin, a):
        y = torch.empty((M, lin.out_features), dtype=torch.bfloat16, device=dev)
        return timed(lambda: G.FP8GEMMScaled(M, lin.out_features, lin.in_features, a.codes.data_ptr(), lin.w.codes.data_ptr(),
                                             y.data_ptr(), 1.0, a.scale_ptr, lin.w.scale_ptr, G.OutBF16, sh))

    hq = quantize(rn(M, Fh, std=1.0))
    t_qkv, t_o, t_gu, t_dn = gemm(blk.qkv, xq), gemm(blk.o, xq), gemm(blk.gate_up, xq), gemm(blk.down, hq)
    hd = d // H
    q3 = [quantize(rn(B * H, S, hd, std=1.0)) for _ in range(3)]
    o = torch.empty((B * H, S, hd), dtype=torch.float16, device=dev)
    t_att = timed(lambda: blk.fa.ForwardEx(q3[0].codes.data_ptr(), q3[1].codes.data_ptr(), q3[2].codes.data_ptr(), o.data_ptr(), 0,
                                           B * H, S, hd, 1, 0, 1 / math.sqrt(hd), 1.0, q3[0].scale_ptr, q3[1].scale_ptr, q3[2].scale_ptr, sh))
    fl_gemm = 2.0 * M * d * (3 * d + d + 3 * Fh)
    fl_att = 2.0 * B * H * S * S * hd
    kern = t_qkv + t_o + t_gu + t_dn + t_att
    print(f"block B={B} S={S} d={d} H={H} F={Fh}: total {total:.3f} ms; FP8 kernels {kern:.3f} ms "
          f"(qkv {t_qkv:.3f}, o {t_o:.3f}, gate+up {t_gu:.3f}, down {t_dn:.3f}, attention {t_att:.3f}); fused glue+quantise {total - kern:.3f} ms; "
          f"same block with torch glue and separate quantiser calls {total_unfused:.3f} ms")
    print(f"GEMM {fl_gemm / (t_qkv + t_o + t_gu + t_dn) / 1e9:.0f} TFLOPS over {fl_gemm / 1e12:.2f} TFLOP; "
          f"attention (causal) {fl_att / t_att / 1e9:.0f} TFLOPS; whole block {(fl_gemm + fl_att) / total / 1e9:.0f} TFLOPS")
    blk.close()


if __name__ == "__main__":
    _main()
