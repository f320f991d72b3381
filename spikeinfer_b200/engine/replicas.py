"""Request sharding across independent per-GPU replicas.

Decode requests are independent units, so multi-GPU serving is one engine replica per GPU (own model
copy, page pool, block allocator and CUDA graphs) with the requests partitioned between them; nothing
crosses GPUs on the data path.  The only collective is the max-reduce of the timing numbers.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_requests(num_requests: int, world_size: int, rank: int) -> range:
    """Contiguous, balanced slice of ``range(num_requests)`` owned by ``rank`` (sizes differ by at most one)."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(num_requests, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def max_over_ranks(values: list[float], device: torch.device | str = "cpu") -> list[float]:
    """Element-wise maximum of ``values`` over all ranks (identity without an initialised process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def aggregate_throughput(units_per_rank: int, seconds_per_rank: float, device: torch.device | str = "cpu") -> float:
    """Whole-job throughput: units all ranks processed divided by the slowest rank's time."""
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    (slowest,) = max_over_ranks([seconds_per_rank], device)
    return units_per_rank * world / slowest
