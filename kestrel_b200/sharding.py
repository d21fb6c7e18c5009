"""Request sharding across GPUs of one box.

The paged-KV path has no exchange step: every GPU owns its KV pool, page table and (optionally)
prefix cache, and serves its own sequences (the reference is single-GPU; replicas are the
multi-GPU form of this path).  What remains is deciding which rank serves which sequence and
combining per-rank measurements -- both host-side, both collective-free on the data path.
"""

from __future__ import annotations

from typing import Optional

import torch


def shard_bounds(n_items: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced split: rank ``r`` serves items ``[lo, hi)``; sizes differ by at most one."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if n_items < 0:
        raise ValueError("n_items must be non-negative")
    lo = rank * n_items // world_size
    hi = (rank + 1) * n_items // world_size
    return lo, hi


def owner_of(item: int, n_items: int, world_size: int) -> int:
    """Rank that serves ``item`` under :func:`shard_bounds`."""
    if not 0 <= item < n_items:
        raise ValueError("item out of range")
    return ((item + 1) * world_size - 1) // n_items


def combine_step_stats(elapsed_ms: float, work_units: float, device: Optional[torch.device] = None,
                       group=None) -> tuple[float, float]:
    """(max over ranks of the time, sum over ranks of the work) -- the whole-job view of a step that
    every rank ran on its own shard.  Without an initialised process group returns the inputs."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return float(elapsed_ms), float(work_units)
    t = torch.tensor([float(elapsed_ms)], dtype=torch.float64, device=device)
    u = torch.tensor([float(work_units)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(u, op=dist.ReduceOp.SUM, group=group)
    return t.item(), u.item()


def gather_rank_stats(values, device: Optional[torch.device] = None, group=None) -> torch.Tensor:
    """Every rank's measurements side by side: ``values`` (a sequence of floats, the same length on every
    rank) -> float64 tensor ``[world, len(values)]`` on the CPU, row ``r`` from rank ``r``.  One all-gather,
    outside any timed region; without an initialised process group a single row."""
    import torch.distributed as dist

    mine = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if not (dist.is_available() and dist.is_initialized()):
        return mine.cpu().view(1, -1)
    rows = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(rows, mine, group=group)
    return torch.stack(rows).cpu()


def whole_job_rate(elapsed_ms: torch.Tensor, work_units: torch.Tensor) -> tuple[float, float, list[float]]:
    """``(slowest rank's time in ms, work of all ranks per second, each rank's own rate per second)`` of a step
    that every rank ran on its own shard: the job is as slow as its slowest rank and did everybody's work."""
    t = float(elapsed_ms.max())
    total = float(work_units.sum())
    own = [float(u) / (float(ms) * 1e-3) if float(ms) > 0 else 0.0 for ms, u in zip(elapsed_ms.tolist(), work_units.tolist())]
    return t, (total / (t * 1e-3) if t > 0 else 0.0), own
