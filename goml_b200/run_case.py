"""Run one kernel of the path a few times on cuda:0 (for profilers and quick checks).

    python -m goml_b200.run_case fa   BH S D CAUSAL ITERS      # fa_forward_train, random e4m3 inputs
    python -m goml_b200.run_case gemm M N K ITERS              # fp8_gemm_scaled, bf16 out
    python -m goml_b200.run_case quant N ITERS                 # fp8_quantize_f32 (scale = amax/448)

torch only allocates the device buffers; every launch goes through the C ABI.
"""
import math
import sys

import torch

from . import fa_forward as F, fp8_gemm as G, quantize as Q


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
    elif kind == "quant":
        n, iters = args
        x = torch.randn(n, device="cuda")
        q = torch.empty(n, dtype=torch.uint8, device="cuda")
        s = torch.zeros(2, device="cuda")
        for _ in range(iters):
            Q.QuantizeF32ToF8E4M3(x.data_ptr(), q.data_ptr(), s.data_ptr(), s.data_ptr() + 4, n, 0)
        torch.cuda.synchronize()
    else:
        raise SystemExit(__doc__)
    print("ok")


if __name__ == "__main__":
    main(sys.argv[1:])
