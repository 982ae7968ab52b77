"""Replica sharding: independent sequences are dealt round-robin to one Executor per GPU.

The path has no exchange step (the reference has no distributed runtime at all), so the
only multi-GPU logic is which rank takes which item and how per-rank timings combine into a
whole-job throughput.
"""
from __future__ import annotations

from typing import List, Sequence, TypeVar

T = TypeVar("T")


def shard(items: Sequence[T], rank: int, world_size: int) -> List[T]:
    """Items `rank, rank + world_size, ...`: every item goes to exactly one rank."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return [items[i] for i in range(rank, len(items), world_size)]


def aggregate_throughput(items_per_rank: Sequence[int], seconds_per_rank: Sequence[float]) -> float:
    """Whole-job items per second: all items over the slowest rank's time."""
    if len(items_per_rank) != len(seconds_per_rank) or not items_per_rank:
        raise ValueError("one item count and one time per rank are required")
    return sum(items_per_rank) / max(seconds_per_rank)
