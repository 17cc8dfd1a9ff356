"""Request-level replicas: one independent engine per GPU, no collective on the data path.

The reference is single-GPU; its process-per-engine pattern (nanoserve/engine_process.py:160-170) is what scaling by
replicas reuses. Nothing is exchanged between replicas while they serve; the only cross-rank communication is the
bookkeeping of a benchmark or a router: a barrier, and the maximum over ranks of each rank's elapsed time.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def max_over_ranks(seconds: list[float], device="cpu") -> list[float]:
    """Element-wise maximum over all ranks of a short list of timings (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(seconds)
    t = torch.tensor(seconds, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def sum_over_ranks(counts: list[float], device="cpu") -> list[float]:
    """Element-wise sum over all ranks of a short list of counts (identity without a process group): replicas serve
    different request streams, so their token counts differ."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(counts)
    t = torch.tensor(counts, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.tolist()


def aggregate_throughput(units_per_rank: int, seconds: float, device="cpu") -> tuple[float, float]:
    """Whole-job throughput of identical replicas: (world_size * units_per_rank / max-over-ranks seconds, that max)."""
    world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
    slowest = max_over_ranks([seconds], device)[0]
    return world * units_per_rank / slowest, slowest


def replica_seed(base_seed: int, rank: int) -> int:
    """Each replica serves its own request stream: a distinct, reproducible seed per rank."""
    return base_seed + 1000003 * rank
