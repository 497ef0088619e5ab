"""Helpers for the GPU parity tests: torch is used for device memory only."""
import numpy as np
import torch


def dev_u8(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint8)).cuda()


def run_gemm(a, b, alpha=None, bf16=True, scale_ptrs=(0, 0), entry="scaled"):
    """C = A.B^T through the C ABI on e4m3 code arrays; returns a numpy float64 array."""
    from goml_b200 import fp8_gemm as G
    M, K = a.shape
    N = b.shape[0]
    ad, bd = dev_u8(a), dev_u8(b)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16 if bf16 else torch.float16, device="cuda")
    if entry == "scaled":
        G.FP8GEMMScaled(M, N, K, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), 1.0 if alpha is None else alpha,
                        scale_ptrs[0], scale_ptrs[1], G.OutBF16 if bf16 else G.OutFP16, 0)
    elif entry == "gemm":
        G.FP8GEMM(M, N, K, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), 1, 0)
    elif entry == "original":
        G.FP8GEMMOriginal(M, N, K, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), 0)
    else:
        G.FP8GEMMSinglesync(M, N, K, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), 0)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    return c.double().cpu().numpy()


def run_attention(ctx, q, k, v, causal=0, window=0, scale=None, v_descale=1.0, entry="train", want_lse=True):
    """Attention through the C ABI on e4m3 code arrays [bh, sl, hd]; returns (O f64, LSE f64 or None)."""
    import math
    bh, sl, hd = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    qd, kd, vd = dev_u8(q), dev_u8(k), dev_u8(v)
    o = torch.zeros((bh, sl, hd), dtype=torch.float16, device="cuda")          # zero-initialised as the
    lse = torch.zeros((bh, sl), dtype=torch.float32, device="cuda") if want_lse else None  # reference callers do
    lp = lse.data_ptr() if want_lse else 0
    if entry == "train":
        ctx.ForwardTrain(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lp, bh, sl, hd, causal, window, scale, 0)
    elif entry == "forward":
        ctx.Forward(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), bh, sl, hd, causal, window, scale, 0)
    else:
        ctx.ForwardEx(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lp, bh, sl, hd, causal, window, scale, v_descale)
    torch.cuda.synchronize()
    ctx.DeviceStatus()
    return o.double().cpu().numpy(), (lse.double().cpu().numpy() if want_lse and entry != "forward" else None)
