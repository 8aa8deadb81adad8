"""Batch sharding of independent sequence states across ranks (one process per GPU).

Every operation on the path is independent across states, so a multi-GPU job partitions the batch into
contiguous shards and runs with no data-path collective; torch.distributed is used only to agree on
timings (max over ranks) and, optionally, to gather outputs.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_states: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [lo, hi) per rank; the first ``n_states % world_size`` ranks take one extra state."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    base, extra = divmod(int(n_states), int(world_size))
    out, lo = [], 0
    for r in range(world_size):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def shard_of(x: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """This rank's rows of a tensor whose leading dimension indexes states (inputs and CPU-staged
    initial states are generated once at full batch and sliced, so results do not depend on the world size)."""
    lo, hi = shard_bounds(x.shape[0], world_size)[rank]
    return x[lo:hi]


def max_over_ranks(value: float, device=None) -> float:
    """A timing as the job sees it: the slowest rank's."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_rows(x: torch.Tensor) -> torch.Tensor:
    """Concatenate every rank's rows (equal or unequal shard sizes) on all ranks, in rank order."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return x
    ws = dist.get_world_size()
    n = torch.tensor([x.shape[0]], dtype=torch.int64, device=x.device)
    sizes = [torch.zeros_like(n) for _ in range(ws)]
    dist.all_gather(sizes, n)
    m = int(max(int(s.item()) for s in sizes))
    pad = torch.zeros((m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    pad[:x.shape[0]] = x
    parts = [torch.zeros_like(pad) for _ in range(ws)]
    dist.all_gather(parts, pad)
    return torch.cat([p[:int(s.item())] for p, s in zip(parts, sizes)], dim=0)
