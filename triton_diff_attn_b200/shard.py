"""(batch*head) sharding across the GPUs of one box.

Every (batch, head) pair is an independent attention problem (the reference indexes everything by
`index_batch_head`, src/kernel.py:53-59); the only cross-head quantity is the scalar d(lambda).
Each rank therefore runs the operator on its own slice with no collective on the data path, and
the per-rank fp32 d(lambda) partials are brought to the host and summed there in fp64.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of `total` units for `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(b: int, h: int, rank: int, world: int) -> Tuple[int, int]:
    """Shard along the batch dimension when it divides evenly (keeps [B,H,N,D] views), else raise."""
    if b % world != 0:
        raise ValueError(f"batch {b} not divisible by world size {world}; shard flat (b*h) instead")
    per = b // world
    return rank * per, (rank + 1) * per


def sum_dlambda_on_host(partial: torch.Tensor, group=None) -> float:
    """Gather every rank's fp32 d(lambda) partial and sum on the host in fp64 (no device collective
    on the hot path).  Works with gloo (CPU tensors) and nccl (CUDA tensors)."""
    val = partial.detach().reshape(1).to(torch.float32)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(val.double().sum())
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    buf = val.cuda() if backend == "nccl" else val.cpu()
    parts: List[torch.Tensor] = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return float(sum(float(p.cpu().double()) for p in parts))
