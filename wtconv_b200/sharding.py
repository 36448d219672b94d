"""Batch sharding of the WTConv forward across ranks (one process per GPU).

Every (sample, channel) plane of the layer is independent (all convolutions are
depthwise: wtconv/wtconv2d.py:23,27, wtconv/util/wavelet.py:65,74), so N GPUs
simply take N contiguous slices of the batch with replicated weights and run the
single-GPU kernels; there is no collective on the data path.  The only optional
exchange is a final all_gather of the outputs (NCCL on GPUs, gloo in the CPU
tests), for callers that want the whole batch on every rank.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the samples rank `rank` owns: contiguous, sizes differ by at most one,
    earlier ranks take the remainder.  Ranks beyond the batch get an empty range."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    base, rem = divmod(batch, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def gather_outputs(y_local: torch.Tensor, batch: int, group=None) -> torch.Tensor:
    """All-gather the per-rank output slices (ragged and empty shards allowed) into the full batch."""
    world = dist.get_world_size(group)
    sizes = [shard_range(batch, world, r) for r in range(world)]
    longest = max(b - a for a, b in sizes)
    pad = torch.zeros((longest,) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
    pad[: y_local.shape[0]] = y_local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)], dim=0)


def max_over_ranks(value: float, device, group=None) -> float:
    """Timing reduction used by the benchmark: a step is as slow as its slowest rank."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
