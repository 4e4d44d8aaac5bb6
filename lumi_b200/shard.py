"""Batch sharding for multi-GPU runs: independent sequences split contiguously over ranks, no
collective on the data path (the token loop has none).  `torch.distributed` is used only for the
start barrier and the max-over-ranks reduction of timings."""
from __future__ import annotations

import os
from typing import Tuple


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Sequences [lo, hi) of `total` owned by `rank`: contiguous blocks, sizes differing by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def waves(n_seq: int, capacity: int):
    """Splits a shard into waves of at most `capacity` resident sequences: [(lo, hi), ...]."""
    if capacity <= 0:
        raise ValueError("capacity must be > 0")
    n_waves = (n_seq + capacity - 1) // capacity
    out = []
    for w in range(n_waves):
        lo, hi = shard_range(n_seq, w, n_waves)
        out.append((lo, hi))
    return out


def env_rank_world() -> Tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def reduce_max_sum(dist, value_max: float, value_sum: float, device=None):
    """(max over ranks of value_max, sum over ranks of value_sum) — the timing rule of the benchmark:
    the slowest rank's device time, the units all ranks processed."""
    import torch
    t = torch.tensor([value_max], dtype=torch.float64, device=device)
    s = torch.tensor([value_sum], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(s, op=dist.ReduceOp.SUM)
    return float(t.item()), float(s.item())
