"""Host-side logic of running the path as independent replicas, one process per GPU.

The reference shards its work by independent 30 s windows (one engine instance per device, no
data exchanged between them), so the multi-GPU form of this path is N replicas and the only
cross-rank traffic is what a measurement needs: a barrier and the maximum elapsed time.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple


def rank_info() -> Tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment (torchrun), 0/0/1 without one."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def init_group(backend: str, world: int, device=None):
    """Join the process group when there is more than one rank; returns torch.distributed or None."""
    if world <= 1:
        return None
    import torch.distributed as dist
    if not dist.is_initialized():
        if device is not None:
            dist.init_process_group(backend, device_id=device)
        else:
            dist.init_process_group(backend)
    return dist


def max_over_ranks(value: float, dist, device=None) -> float:
    """The slowest rank's figure: a multi-GPU time is the maximum over ranks, never one rank's own."""
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rate(units_per_rank_per_step: float, world: int, seconds_per_step: float) -> float:
    """Aggregate throughput of N replicas doing the same per-rank work (weak scaling)."""
    return world * units_per_rank_per_step / seconds_per_step


def shard_rows(total_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the rows rank owns when a fixed job is cut across replicas (whole rows,
    the first `total_rows % world` ranks take one extra)."""
    base, extra = divmod(total_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)
