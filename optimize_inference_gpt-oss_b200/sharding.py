"""Data-parallel split of a token batch over the GPUs of one box.

Rows are independent, so the path shards with no exchange step: every GPU holds its own
copy of the tables and a contiguous range of the batch, the split the reference engine
uses for its replicas (gpu_engine.hpp:914, 928-929: contiguous request shares per group).
The only cross-rank traffic is bookkeeping outside the data path: a barrier and a max over
the per-rank step times.
"""
from __future__ import annotations


def shard_range(total: int, world: int, rank: int, granule: int = 1) -> tuple[int, int]:
    """[begin, end) of the rows rank `rank` of `world` owns out of `total` rows.

    Ranges are contiguous, ordered by rank, cover [0, total) exactly, and start on a
    multiple of `granule` (e.g. the sequence length, so a sequence never straddles two
    GPUs); the first (units mod world) ranks get one unit more.
    """
    if world <= 0 or not 0 <= rank < world or total < 0 or granule <= 0:
        raise ValueError((total, world, rank, granule))
    if total % granule:
        raise ValueError(f"{total} rows is not a whole number of granules of {granule}")
    units = total // granule
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * granule, end * granule


def max_over_ranks(value: float, dist=None) -> float:
    """The slowest rank's time: all-reduce(max) over the default process group (any
    backend), or `value` itself without one."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, dist=None) -> float:
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
