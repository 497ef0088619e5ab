"""Shape sweep of the FP8 attention forward and the FP8 GEMM on cuda:0 (CUDA-event timing).

    python tests/perf/sweep.py [attn] [gemm]

Attention: hd in {64,128}, S in {1024,4096,16384,32768}, H=32, B chosen so that B*S = 65536, causal and
non-causal.  GEMM: squares 1024..16384 and skinny M in {16,128} with N=K=8192, bf16 output.
FLOP conventions: attention 4*BH*S^2*D (causal: half); GEMM 2*M*N*K.  Prints one line per shape.
"""
import math
import sys

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from goml_b200 import fa_forward as F, fp8_gemm as G  # noqa: E402


def _time(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def attention_sweep():
    ctx = F.FACreate()
    for hd in (128, 64):
        for sl in (1024, 4096, 16384, 32768):
            bh = 32 * (65536 // sl)
            q, k, v = (torch.randn(bh, sl, hd, device="cuda").to(torch.float8_e4m3fn) for _ in range(3))
            o = torch.empty(bh, sl, hd, dtype=torch.float16, device="cuda")
            lse = torch.empty(bh, sl, dtype=torch.float32, device="cuda")
            for causal in (0, 1):
                ms = _time(lambda: ctx.ForwardTrain(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                                    bh, sl, hd, causal, 0, 1 / math.sqrt(hd)), iters=5)
                fl = 4.0 * bh * sl * sl * hd / (2 if causal else 1)
                print(f"attn hd={hd:3d} BH={bh:4d} S={sl:5d} causal={causal}  {ms:8.3f} ms  {fl / ms / 1e9:8.1f} TFLOPS", flush=True)
            del q, k, v, o, lse
    ctx.DeviceStatus()
    ctx.Destroy()


def gemm_sweep():
    shapes = [(n, n, n) for n in (1024, 2048, 4096, 8192, 16384)] + [(16, 8192, 8192), (128, 8192, 8192)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(N, K, device="cuda").to(torch.float8_e4m3fn)
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        ms = _time(lambda: G.FP8GEMMScaled(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, 0, 0, G.OutBF16, 0),
                   iters=20 if M * N * K < 2 ** 38 else 5)
        fl = 2.0 * M * N * K
        gbs = (M * K + N * K + 2 * M * N) / ms / 1e6
        print(f"gemm {M:5d}x{N:5d}x{K:5d}  {ms:8.4f} ms  {fl / ms / 1e9:8.1f} TFLOPS  {gbs:8.1f} GB/s algorithmic", flush=True)
    assert G.device_status() == 0


if __name__ == "__main__":
    what = sys.argv[1:] or ["attn", "gemm"]
    if "attn" in what:
        attention_sweep()
    if "gemm" in what:
        gemm_sweep()
