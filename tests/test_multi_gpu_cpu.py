"""Host-side sharding logic of the N>1 path, run as two gloo ranks on CPU.
The per-rank compute is the oracle GEMM (a stand-in for the kernel, which needs
a GPU); what is under test is the partition and the optional all-gather."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from goml_b200 import multi_gpu as MG


def test_partitions_cover_exactly_once():
    for total in (1, 7, 16, 128, 129, 2048):
        for ws in (1, 2, 3, 4, 8):
            spans = [MG.shard_heads(total, ws, r) for r in range(ws)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(ws - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    for M in (16, 128, 1000, 8192, 16384):
        for ws in (1, 2, 4, 8):
            spans = [MG.shard_rows(M, ws, r) for r in range(ws)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(b % 128 == 0 for b, _ in spans if b < M)
    assert MG.shard_rows(16384, 8, 3) == (6144, 8192)   # C4: one batch element (2048 tokens) per GPU
    assert MG.shard_heads(128, 8, 7) == (112, 128)       # C3: 16 heads per GPU


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, ws, port, M, N, K, q):
    import oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    a, b = O.harness_gemm_inputs(M, N, K)
    r0, r1 = MG.shard_rows(M, ws, rank)
    local = torch.from_numpy(O.gemm_f64(a[r0:r1], b)).to(torch.bfloat16)  # rank-local rows, replicated B
    full = MG.allgather_rows(local, M, ws, rank)
    into = MG.allgather_rows_into(torch.empty((M, N), dtype=torch.bfloat16), local, M, ws, rank)    # unequal blocks: padded path
    assert torch.equal(into, full)
    M2 = 512                                                                                       # equal blocks: one direct all-gather
    a2, b2 = O.harness_gemm_inputs(M2, N, K)
    s0, s1 = MG.shard_rows(M2, ws, rank)
    local2 = torch.from_numpy(O.gemm_f64(a2[s0:s1], b2)).to(torch.bfloat16)
    full2 = MG.allgather_rows_into(torch.empty((M2, N), dtype=torch.bfloat16), local2, M2, ws, rank)
    assert torch.equal(full2, torch.from_numpy(O.gemm_f64(a2, b2)).to(torch.bfloat16))
    h0, h1 = MG.shard_heads(6, ws, rank)
    qa, ka, va = O.harness_attention_inputs(6, 64, 64)
    o_local, _ = O.attention_f64(qa[h0:h1], ka[h0:h1], va[h0:h1])  # heads are independent: no exchange
    if rank == 0:
        q.put((full.float().numpy(), o_local, (h0, h1)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gloo_sharded_gemm_and_attention():
    import oracle as O
    M, N, K = 300, 64, 64   # 3 row tiles over 2 ranks -> uneven blocks (256 + 44)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, N, K, q)) for r in range(2)]
    for p in procs:
        p.start()
    full, o_local, (h0, h1) = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    a, b = O.harness_gemm_inputs(M, N, K)
    want = torch.from_numpy(O.gemm_f64(a, b)).to(torch.bfloat16).float().numpy()
    assert full.shape == (M, N) and np.array_equal(full, want)
    qa, ka, va = O.harness_attention_inputs(6, 64, 64)
    o_all, _ = O.attention_f64(qa, ka, va)
    assert np.array_equal(o_local, o_all[h0:h1])
