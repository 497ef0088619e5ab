"""Run one kernel of the path a few times on cuda:0 (for profilers and quick checks).

    python tests/perf/run_case.py fa   BH S D CAUSAL ITERS      # fa_forward_train, random e4m3 inputs
    python tests/perf/run_case.py gemm M N K ITERS              # fp8_gemm_scaled, bf16 out
    python tests/perf/run_case.py blockdec B S D_MODEL H F ITERS  # one decode step of the whole FP8 block against a cache of S keys
    python tests/perf/run_case.py decstep B HQ HKV S D ITERS    # new token's RoPE + quantise + cache append, then fa_decode
    python tests/perf/run_case.py gemm8 M N K ITERS             # bf16-out and e4m3-out epilogues timed side by side
    python tests/perf/run_case.py gemm_mx M N K ITERS           # block-scaled GEMM (fp8_gemm_mx) beside the per-tensor kernel, with timing
    python tests/perf/run_case.py quant N ITERS                 # fp8_quantize_f32 (scale = amax/448)
    python tests/perf/run_case.py glue B S D H F ITERS          # the six libfp8block.so ops of one decoder block, with timings
    python tests/perf/run_case.py decode B HQ HKV S D ITERS [PAGE]   # fa_decode: one token per sequence, e4m3 KV cache of S keys, with timing; PAGE: paged cache
    python tests/perf/run_case.py block B S D H F ITERS         # one fused FP8 decoder block (goml_b200.nn), random-init weights

torch only allocates the device buffers; every launch goes through the C ABI.
"""
import math
import sys

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from goml_b200 import block_glue as BG, fa_forward as F, fp8_gemm as G, quantize as Q  # noqa: E402


def main(argv):
    kind, args = argv[0], [int(x) for x in argv[1:]]
    if kind == "fa":
        bh, sl, hd, causal, iters = args
        ctx = F.FACreate()
        g = torch.Generator(device="cuda").manual_seed(0)
        q, k, v = (torch.randn(bh, sl, hd, device="cuda", generator=g).mul_(0.5).to(torch.float8_e4m3fn) for _ in range(3))
        o = torch.empty(bh, sl, hd, dtype=torch.float16, device="cuda")
        lse = torch.empty(bh, sl, dtype=torch.float32, device="cuda")
        for _ in range(iters):
            ctx.ForwardTrain(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), bh, sl, hd, causal, 0, 1 / math.sqrt(hd))
        torch.cuda.synchronize()
        ctx.DeviceStatus()
    elif kind == "gemm":
        M, N, K, iters = args
        a = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(N, K, device="cuda").to(torch.float8_e4m3fn)
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        for _ in range(iters):
            G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, 0, 0, G.OutBF16, 0)
        torch.cuda.synchronize()
        assert G.device_status() == 0
    elif kind == "gemm_mx":
        M, N, K, iters = args
        xa, xb = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda")
        a, b = torch.empty(M, K, dtype=torch.uint8, device="cuda"), torch.empty(N, K, dtype=torch.uint8, device="cuda")
        sa = torch.empty(Q.mx_scale_bytes(M, K), dtype=torch.uint8, device="cuda")
        sb = torch.empty(Q.mx_scale_bytes(N, K), dtype=torch.uint8, device="cuda")
        Q.QuantizeMXF32(xa.data_ptr(), a.data_ptr(), sa.data_ptr(), M, K)
        Q.QuantizeMXF32(xb.data_ptr(), b.data_ptr(), sb.data_ptr(), N, K)
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        runs = {
            "block-scaled (fp8_gemm_mx)": lambda: G.FP8GEMMMX(M, N, K, a.data_ptr(), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), c.data_ptr(), 1.0, G.OutBF16),
            "per-tensor (fp8_gemm_scaled)": lambda: G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, 0, 0, G.OutBF16, 0),
        }
        for name, fn in runs.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            print(f"{name}: {M}x{N}x{K}  {ms * 1e3:.1f} us  {2.0 * M * N * K / ms / 1e9:.0f} TFLOPS")
        assert G.mx_device_status() == 0 and G.device_status() == 0
    elif kind == "gemm8":
        # the e4m3-output epilogue beside the bf16 one on the same operands: ms and TFLOPS of each
        M, N, K, iters = args
        a = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(N, K, device="cuda").to(torch.float8_e4m3fn)
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        d = torch.empty(M, N, dtype=torch.uint8, device="cuda")
        s = torch.tensor([1.0, 1.0, 448.0 / (6.0 * K ** 0.5), 0.0], device="cuda")
        runs = {
            "bf16 out": lambda: G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, 0, 0, G.OutBF16, 0),
            "e4m3 out + amax": lambda: G.FP8GEMMFP8Out(M, N, K, a.data_ptr(), b.data_ptr(), d.data_ptr(), 1.0, s.data_ptr(),
                                                       s.data_ptr() + 4, s.data_ptr() + 8, s.data_ptr() + 12),
        }
        for name, fn in runs.items():
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            print(f"gemm {M}x{N}x{K} {name}: {ms:.4f} ms, {2.0 * M * N * K / ms / 1e9:.0f} TFLOPS")
        assert G.device_status() == 0 and s[3].item() > 0
    elif kind == "quant":
        n, iters = args
        x = torch.randn(n, device="cuda")
        q = torch.empty(n, dtype=torch.uint8, device="cuda")
        s = torch.zeros(2, device="cuda")
        for _ in range(iters):
            Q.QuantizeF32ToF8E4M3(x.data_ptr(), q.data_ptr(), s.data_ptr(), s.data_ptr() + 4, n, 0)
        torch.cuda.synchronize()
    elif kind == "block":
        from goml_b200 import nn
        B, S, d, H, Fh, iters = args
        g = torch.Generator(device="cuda").manual_seed(4)
        rn = lambda *shape, std=0.02: torch.randn(*shape, generator=g, device="cuda") * std
        blk = nn.FP8DecoderBlock(d, H, Fh, rn(3 * d, d), rn(d, d), rn(2 * Fh, d), rn(d, Fh), torch.ones(d, device="cuda"), torch.ones(d, device="cuda"))
        x = rn(B * S, d, std=1.0)
        blk(x, B, S)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            y = blk(x, B, S)
        e1.record()
        torch.cuda.synchronize()
        blk.fa.DeviceStatus()
        assert G.device_status() == 0 and bool(torch.isfinite(y).all())
        print(f"block B={B} S={S} d={d} H={H} F={Fh}: {e0.elapsed_time(e1) / iters:.3f} ms per block")
        blk.close()
    elif kind == "decode":
        # optional 7th argument: page size of a paged cache (pages of every sequence scattered over the pool)
        B, hq, hkv, S, D, iters = args[:6]
        page = args[6] if len(args) > 6 else 0
        ctx = F.FACreate()
        g = torch.Generator(device="cuda").manual_seed(0)
        q = torch.randn(B, hq, D, device="cuda", generator=g).mul_(0.5).to(torch.float8_e4m3fn)
        kc, vc = (torch.randn(B, hkv, S, D, device="cuda", generator=g).mul_(0.5).to(torch.float8_e4m3fn) for _ in range(2))
        o = torch.empty(B, hq, D, dtype=torch.float16, device="cuda")
        if page:
            assert S % page == 0
            per_seq = S // page
            # the same bytes seen as a pool [B * per_seq, hkv, page, D]; a random table spreads each sequence over it
            table = torch.randperm(B * per_seq, generator=g, device="cuda").to(torch.int32).view(B, per_seq).contiguous()
            fn = lambda: ctx.Decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), 0, 0, B, hq, hkv, D, 0, S, 1 / math.sqrt(D),
                                    block_table=table.data_ptr(), page_size=page, max_pages_per_seq=per_seq, num_pages=B * per_seq)
        else:
            fn = lambda: ctx.Decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), 0, 0, B, hq, hkv, D, S, S, 1 / math.sqrt(D))
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ctx.DeviceStatus()
        us = e0.elapsed_time(e1) / iters * 1e3
        nbytes = 2 * B * hkv * S * D
        print(f"decode B={B} Hq={hq} Hkv={hkv} S={S} D={D}{f' page={page}' if page else ''}: {us:8.1f} us   {nbytes / us / 1e3:7.0f} GB/s of the KV cache ({nbytes / 1e6:.0f} MB)")
    elif kind == "blockdec":
        # one decode step of the whole block (one new token per sequence) against a cache of S keys per sequence
        from goml_b200 import nn
        B, S, d, H, Fh, iters = args
        g = torch.Generator(device="cuda").manual_seed(4)
        rn = lambda *shape, std=0.02: torch.randn(*shape, generator=g, device="cuda") * std
        blk = nn.FP8DecoderBlock(d, H, Fh, rn(3 * d, d), rn(d, d), rn(2 * Fh, d), rn(d, Fh), torch.ones(d, device="cuda"), torch.ones(d, device="cuda"))
        cache = nn.FP8KVCache(B, H, S + 2 * iters + 16, d // H)
        cache.k[:, :, :S].copy_(torch.randn(B, H, S, d // H, generator=g, device="cuda").to(torch.float8_e4m3fn).view(torch.uint8))
        cache.v[:, :, :S].copy_(torch.randn(B, H, S, d // H, generator=g, device="cuda").to(torch.float8_e4m3fn).view(torch.uint8))
        cache.lens.fill_(S)
        x = rn(B, d, std=1.0)
        for _ in range(3):
            y = blk.decode_step(x, cache)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            y = blk.decode_step(x, cache)
        e1.record()
        torch.cuda.synchronize()
        blk.fa.DeviceStatus()
        assert G.device_status() == 0 and bool(torch.isfinite(y).all()) and int(cache.lens[0]) == S + 3 + iters
        us = e0.elapsed_time(e1) / iters * 1e3
        nbytes = d * (3 * d + d + 3 * Fh) + 2 * B * H * S * (d // H)          # weights once + the K and V cache once
        print(f"block decode step B={B} cache S={S} d={d} H={H} F={Fh}: {us:8.1f} us per step, {nbytes / us / 1e3:6.0f} GB/s "
              f"of weights + cache ({nbytes / 1e6:.0f} MB)")
        # the same step captured once in a CUDA graph and replayed: the ~20 launches of a step cost no host time
        cache.lens.fill_(S)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            blk.decode_step(x, cache)                                          # warm-up on the capture stream
            side.synchronize()
            cache.lens.fill_(S)
            with torch.cuda.graph(graph, stream=side):
                yg = blk.decode_step(x, cache)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        blk.fa.DeviceStatus()
        assert G.device_status() == 0 and bool(torch.isfinite(yg).all()) and int(cache.lens[0]) == S + 2 + iters
        usg = e0.elapsed_time(e1) / iters * 1e3
        print(f"block decode step B={B} cache S={S} replayed from a CUDA graph: {usg:8.1f} us per step, {nbytes / usg / 1e3:6.0f} GB/s")
        blk.close()
    elif kind == "decstep":
        # one decode step's attention part: RoPE + quantise + cache append of the new token, then fa_decode
        from goml_b200 import block_glue as BG
        B, hq, hkv, S, D, iters = args
        ctx = F.FACreate()
        g = torch.Generator(device="cuda").manual_seed(0)
        kc, vc = (torch.randn(B, hkv, S, D, device="cuda", generator=g).mul_(0.5).to(torch.float8_e4m3fn) for _ in range(2))
        qkv = torch.randn(B, (hq + 2 * hkv) * D, device="cuda", generator=g).bfloat16()
        cos, sin = torch.empty(S, D // 2, device="cuda"), torch.empty(S, D // 2, device="cuda")
        BG.RopeTable(cos.data_ptr(), sin.data_ptr(), S, D, 10000.0)
        pos = torch.full((B,), S - 1, dtype=torch.int32, device="cuda")
        lens = torch.zeros(B, dtype=torch.int32, device="cuda")
        q = torch.empty(B, hq, D, dtype=torch.uint8, device="cuda")
        o = torch.empty(B, hq, D, dtype=torch.float16, device="cuda")
        sc = torch.tensor([0.0, 0.0, 1.0, 1.0], device="cuda")
        def append():
            BG.DecodeRopeAppend(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), q.data_ptr(), sc.data_ptr(), sc.data_ptr() + 4,
                                kc.data_ptr(), vc.data_ptr(), sc.data_ptr() + 8, sc.data_ptr() + 12, B, hq, hkv, D, S, S, seq_lens_out=lens.data_ptr())
        def attend():
            ctx.Decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), 0, lens.data_ptr(), B, hq, hkv, D, S, 0, 1 / math.sqrt(D), 1.0,
                       scale_q_dev=sc.data_ptr())
        for name, fn in (("append", append), ("append + attend", lambda: (append(), attend()))):
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            print(f"decstep B={B} Hq={hq} Hkv={hkv} S={S} D={D} {name}: {e0.elapsed_time(e1) / iters * 1e3:8.1f} us")
        ctx.DeviceStatus()
        assert bool(torch.isfinite(o.float()).all()) and int(lens[0]) == S
    elif kind == "glue":
        B, S, d, H, Fh, iters = args
        T, hd, dev = B * S, d // H, "cuda"
        x = torch.randn(T, d, device=dev)
        res = torch.randn(T, d, device=dev).bfloat16()
        gamma = torch.ones(d, device=dev)
        q = torch.empty(T, d, dtype=torch.uint8, device=dev)
        sa = torch.zeros(8, device=dev)
        rstd = torch.empty(T, device=dev)
        qkv = torch.randn(T, 3 * d, device=dev).bfloat16()
        cos = torch.empty(S, hd // 2, device=dev)
        sin = torch.empty_like(cos)
        qc, kc, vc = (torch.empty(B * H, S, hd, dtype=torch.uint8, device=dev) for _ in range(3))
        o = torch.randn(B * H, S, hd, device=dev).half()
        gu = torch.randn(T, 2 * Fh, device=dev).bfloat16()
        hq = torch.empty(T, Fh, dtype=torch.uint8, device=dev)
        BG.RopeTable(cos.data_ptr(), sin.data_ptr(), S, hd, 10000.0)
        p = lambda t: t.data_ptr()
        ops = {   # name -> (call, bytes if every input were read once)
            "rmsnorm_quantize": (lambda: BG.RMSNormQuantize(p(x), 0, 0, p(gamma), p(q), p(sa), p(sa) + 4, p(rstd), T, d, 1e-5), T * d * 5),
            "rmsnorm_quantize+residual": (lambda: BG.RMSNormQuantize(p(x), p(res), p(x), p(gamma), p(q), p(sa), p(sa) + 4, p(rstd), T, d, 1e-5), T * d * 11),
            "rope_quantize_qkv": (lambda: BG.RopeQuantizeQKV(p(qkv), p(cos), p(sin), p(qc), p(kc), p(vc), p(sa), p(sa) + 12, B, S, H, hd), T * d * 9),
            "permute_quantize_heads": (lambda: BG.PermuteQuantizeHeads(p(o), p(q), p(sa), p(sa) + 4, B, S, H, hd), T * d * 3),
            "swiglu_quantize": (lambda: BG.SwiGLUQuantize(p(gu), p(hq), p(sa), p(sa) + 4, T, Fh), T * Fh * 5),
            "residual_add": (lambda: BG.ResidualAdd(p(x), p(res), T * d), T * d * 10),
        }
        for name, (fn, nbytes) in ops.items():
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / iters * 1e3
            print(f"{name:28s} {us:8.1f} us   {nbytes / us / 1e3:7.0f} GB/s of single-read bytes")
    else:
        raise SystemExit(__doc__)
    print("ok")


if __name__ == "__main__":
    main(sys.argv[1:])
