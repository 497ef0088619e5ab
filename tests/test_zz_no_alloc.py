"""The allocation-free attention entry point (fa_forward_noalloc), collected last.

It serves callers that may not call the allocator (a framework that reserved the
whole GPU, a process with a frozen memory map): its scratch is a fixed array inside
the library.  The test calls it through the C ABI twice in a row on different
problems — the shared scratch keeps the first call's contents, which must not leak
into the second — and compares each result with the regular entry point's.
"""
import math

import numpy as np
import pytest
import torch

import oracle as O
from tests.gpu_util import dev_u8

pytestmark = pytest.mark.gpu


def _regular(ctx, qd, kd, vd, bh, sl, hd, causal, window, scale, vds):
    o = torch.zeros((bh, sl, hd), dtype=torch.float16, device="cuda")
    lse = torch.zeros((bh, sl), dtype=torch.float32, device="cuda")
    ctx.ForwardEx(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), bh, sl, hd, causal, window, scale, vds)
    torch.cuda.synchronize()
    return o, lse


def _noalloc(qd, kd, vd, bh, sl, hd, causal, window, scale, vds):
    from goml_b200 import fa_forward as F
    o = torch.zeros((bh, sl, hd), dtype=torch.float16, device="cuda")
    lse = torch.zeros((bh, sl), dtype=torch.float32, device="cuda")
    F.FAForwardNoAlloc(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), bh, sl, hd, causal, window, scale, vds)
    torch.cuda.synchronize()
    return o, lse


def test_two_calls_in_a_row_match_the_regular_entry_point(fa_ctx):
    cases = [(6, 1000, 128, 1, 0), (3, 280, 64, 0, 0)]   # second problem is smaller: stale scratch lies beyond it
    for n, (bh, sl, hd, causal, window) in enumerate(cases):
        (q, sq, _), (k, sk, _), (v, sv, _) = [O.quantize_f32(O.seeded_normal(t, (bh, sl, hd), config=f"noalloc{n}")) for t in "QKV"]
        scale = float(sq) * float(sk) / math.sqrt(hd)
        qd, kd, vd = dev_u8(q), dev_u8(k), dev_u8(v)
        o1, l1 = _noalloc(qd, kd, vd, bh, sl, hd, causal, window, scale, float(sv))
        o0, l0 = _regular(fa_ctx, qd, kd, vd, bh, sl, hd, causal, window, scale, float(sv))
        # same kernels, same inputs: within the attention tolerance (max-abs 2e-2, mean-rel 1e-2) — in fact identical
        maxabs, meanrel = O.error_stats(o1.double().cpu().numpy(), o0.double().cpu().numpy())
        assert maxabs <= 2e-2 and meanrel <= 1e-2
        assert torch.equal(o1, o0) and torch.equal(l1, l0)
        ref, lref = O.attention_f64(q, k, v, causal, window, scale, float(sv))
        maxabs, meanrel = O.error_stats(o1.double().cpu().numpy(), ref)
        assert maxabs <= 2e-2 and meanrel <= 1e-2
        assert np.abs(l1.double().cpu().numpy() - lref).max() <= 5e-3


def test_problem_larger_than_the_fixed_scratch_is_rejected(cuda, built_libs):
    from goml_b200 import fa_forward as F
    buf = torch.zeros(1 << 12, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    bh, sl, hd = 17, 8192, 128                      # 17 * 8192 * 128 > 16 Mi elements
    assert bh * sl * hd > F.NOALLOC_MAX_ELEMS
    with pytest.raises(F.FAError) as e:
        F.FAForwardNoAlloc(p, p, p, p, 0, bh, sl, hd, 0, 0, 1.0)   # rejected before any memory is touched
    assert e.value.status == F.FA_ERR_UNSUPPORTED_SHAPE and "exceeds the fixed scratch" in str(e.value)
    with pytest.raises(F.FAError) as e:
        F.FAForwardNoAlloc(0, p, p, p, 0, 1, 64, 128, 0, 0, 1.0)
    assert e.value.status == F.FA_ERR_INVALID_ARG
