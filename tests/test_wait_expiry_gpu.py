"""The failure branch of the bounded waits, run without faulting or hanging anything.

Every mbarrier wait in the kernels is bounded; when the bound is hit the waiter records a code, the thread block
drains and returns, and the host reads the code through *_device_status.  Here a one-warp kernel in each library waits
with a 1 ms budget on a barrier that nothing ever arrives at (no TMA, no tensor memory, nothing in flight), so the wait
must run out: the kernel has to return, the status call has to report the code once and then be clear again, and the
library has to keep working on the same context afterwards.
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests.gpu_util import run_gemm

pytestmark = pytest.mark.gpu


def test_gemm_wait_expiry_is_reported_and_cleared(cuda, built_libs):
    from goml_b200 import fp8_gemm as G
    assert G.device_status() == 0
    G.SelftestWaitExpiry()
    assert G.device_status() == 0x1F0          # the kernel returned (this call synchronises) and latched its code
    assert G.device_status() == 0              # read-and-clear
    a, b = O.harness_gemm_inputs(128, 128, 128)
    got = run_gemm(a, b, bf16=False, entry="gemm")          # the context is still usable
    assert np.array_equal(got, O.round_fp16(O.gemm_f32(a, b)).astype(np.float64))


def test_attention_wait_expiry_is_reported_and_cleared(fa_ctx):
    from goml_b200 import fa_forward as F
    fa_ctx.DeviceStatus()
    fa_ctx.SelftestWaitExpiry()
    with pytest.raises(F.FAError) as e:
        fa_ctx.DeviceStatus()
    assert e.value.status == F.FA_ERR_INTERNAL and "0x2f0" in str(e.value)
    fa_ctx.DeviceStatus()                      # cleared
    fa_ctx.SelftestWaitExpiry()
    assert F.FANoAllocDeviceStatus() == 0x2F0  # the context-free reader sees the same word
    assert F.FANoAllocDeviceStatus() == 0
    torch.cuda.synchronize()
