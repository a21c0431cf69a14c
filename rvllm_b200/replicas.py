"""Replica-parallel bookkeeping: the decode path has no cross-GPU exchange (the reference has no
tensor/pipeline parallelism at all), so N GPUs run N independent replicas and requests are split
between them.  These helpers are the whole of the multi-GPU logic: who serves which requests, and
how per-rank timings become one job-level number (slowest rank wins)."""
from __future__ import annotations


def split_requests(total: int, world: int, rank: int) -> range:
    """Contiguous, even split of `total` request slots; the first total % world ranks take one more."""
    if world <= 0 or not (0 <= rank < world) or total < 0:
        raise ValueError("bad replica split")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def job_seconds(dist, seconds: float, device=None) -> float:
    """Max over ranks of a rank-local duration (all ranks get the result)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(seconds)
    import torch

    t = torch.tensor([seconds], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(dist, units_this_rank: int, seconds: float, device=None) -> float:
    """Whole-job units per second: units of every rank divided by the slowest rank's time."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return units_this_rank / seconds
    import torch

    u = torch.tensor([float(units_this_rank)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return float(u.item()) / job_seconds(dist, seconds, device)
