"""Multi-GPU sharding of the FP8 attention / GEMM path: one process per GPU.

goml itself is single-device (its Backend never sets a device index,
backend/cuda/cuda..go:27,67); this module is the per-device context/stream
manager plus the partition rules the path needs:

* attention shards the batch*head axis contiguously (every head is
  independent) — no collective;
* the GEMM shards M in whole 128-row tiles, B (the weight) is replicated — no
  collective on the hot path; ``allgather_rows`` is the optional NCCL
  all-gather of the C row blocks for callers that need the full C everywhere.

The partition helpers are pure functions (tested on CPU); ``DeviceContext``
owns the FA context and a stream for one GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

GEMM_TILE_M = 128


def shard_heads(batch_heads: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) slice of the batch*head axis owned by `rank`.

    Remainders go to the lowest ranks, so sizes differ by at most one head."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    base, rem = divmod(batch_heads, world_size)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_rows(M: int, world_size: int, rank: int, tile: int = GEMM_TILE_M) -> tuple[int, int]:
    """Contiguous [begin, end) block of GEMM rows owned by `rank`, cut on tile boundaries."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    tiles = (M + tile - 1) // tile
    tb, te = shard_heads(tiles, world_size, rank)
    return min(tb * tile, M), min(te * tile, M)


def shard_cols(N: int, world_size: int, rank: int, tile: int = 256) -> tuple[int, int]:
    """Column partition for skinny-M GEMMs (M smaller than one tile per rank):
    B rows / C columns are split instead, A is replicated."""
    return shard_rows(N, world_size, rank, tile)


def allgather_rows(local_c, M: int, world_size: int, rank: int, group=None):
    """All-gather the row blocks of C (any torch dtype) into the full [M, N] matrix.

    Uses torch.distributed (NCCL over NVLink on GPUs, gloo on CPU).  Row blocks
    may differ in size by one tile, so ranks exchange padded blocks and trim."""
    import torch
    import torch.distributed as dist

    N = local_c.shape[1]
    spans = [shard_rows(M, world_size, r) for r in range(world_size)]
    max_rows = max(e - b for b, e in spans)
    padded = torch.zeros((max_rows, N), dtype=local_c.dtype, device=local_c.device)
    padded[: local_c.shape[0]] = local_c
    out = [torch.empty_like(padded) for _ in range(world_size)]
    dist.all_gather(out, padded, group=group)
    return torch.cat([out[r][: spans[r][1] - spans[r][0]] for r in range(world_size)], dim=0)


def allgather_rows_into(full_c, local_c, M: int, world_size: int, rank: int, group=None):
    """The same exchange into a caller-owned [M, N] matrix, with no staging when the row blocks are equal
    (M a multiple of world_size * 128, the usual case): one NCCL all-gather writes every rank's block straight
    to its place in `full_c`.  Unequal blocks fall back to the padded exchange of ``allgather_rows``.  Returns `full_c`."""
    import torch.distributed as dist

    spans = [shard_rows(M, world_size, r) for r in range(world_size)]
    rows = spans[0][1] - spans[0][0]
    if all(e - b == rows for b, e in spans) and rows * world_size == M and local_c.is_contiguous() and full_c.is_contiguous():
        if local_c.shape[0] != rows:
            raise ValueError("local block does not match this rank's row span")
        dist.all_gather_into_tensor(full_c, local_c, group=group)
        return full_c
    full_c.copy_(allgather_rows(local_c, M, world_size, rank, group))
    return full_c


@dataclass
class DeviceContext:
    """Per-GPU state: device index, a CUDA stream and an FA context created on it."""
    device: int
    stream: object = None
    fa: object = None

    @classmethod
    def create(cls, device: int) -> "DeviceContext":
        import torch
        from . import fa_forward

        torch.cuda.set_device(device)
        stream = torch.cuda.Stream(device=device)
        return cls(device=device, stream=stream, fa=fa_forward.FACreate())

    def close(self) -> None:
        if self.fa is not None:
            self.fa.Destroy()
            self.fa = None
