"""The sharded GEMM and its optional all-gather on real GPUs, one process per GPU over NCCL.

Needs two GPUs in the machine; with fewer the test is skipped (the partition rules and the exchange itself are covered
on CPU with two gloo ranks in tests/test_multi_gpu_cpu.py).  Each rank computes its own 128-row-tile block of
C = alpha * A . B^T through the C ABI (B replicated, no collective), the blocks are all-gathered with NCCL into the
full matrix on every rank, and rank 0 checks sampled rows of the gathered matrix against the oracle and that every
rank holds the same bytes.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["GOML_B200_ROOT"])
import oracle as O
from goml_b200 import fp8_gemm as G, multi_gpu as MG
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
for M, N, K in [(1024, 512, 256), (640, 384, 128)]:          # equal blocks; unequal blocks (5 tiles over 2 ranks)
    g = torch.Generator(device="cuda").manual_seed(11)        # same seed on every rank: the global A and B
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.5).to(torch.float8_e4m3fn)
    r0, r1 = MG.shard_rows(M, world, rank)
    mine = torch.empty((r1 - r0, N), dtype=torch.bfloat16, device="cuda")
    G.FP8GEMMScaled(r1 - r0, N, K, a[r0:r1].contiguous().data_ptr(), b.data_ptr(), mine.data_ptr(), 0.125, 0, 0, G.OutBF16, 0)
    full = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    MG.allgather_rows_into(full, mine, M, world, rank)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    assert torch.equal(full[r0:r1], mine)
    digest = full.view(torch.int16).to(torch.int64).sum().reshape(1)
    all_d = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(all_d, digest)
    assert all(int(d) == int(all_d[0]) for d in all_d)        # every rank holds the same matrix
    if rank == 0:
        ref = O.gemm_f64(a.view(torch.uint8).cpu().numpy(), b.view(torch.uint8).cpu().numpy(), 0.125)
        rms = float(np.sqrt(np.mean(ref ** 2)))
        maxabs, meanrel = O.error_stats(full.double().cpu().numpy() / rms, ref / rms)
        assert maxabs <= 2e-2 and meanrel <= 1e-2, (maxabs, meanrel)
dist.barrier()
dist.destroy_process_group()
if rank == 0:
    print("ALLGATHER_OK")
"""


def test_row_sharded_gemm_and_nccl_allgather_on_two_gpus(cuda, built_libs, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, GOML_B200_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29731", str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "ALLGATHER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
