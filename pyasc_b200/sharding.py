"""Splitting the five workloads over the GPUs of one node.

The reference is single-device (it has no collective of any kind), and none of these computations
has an exchange step: every kernel is a map over independent units (element ranges, softmax rows,
GEMM row blocks, attention batch x heads).  One process drives one GPU (``torch.distributed``, NCCL
on GPUs, gloo in the CPU tests); each rank runs the ordinary single-GPU kernel on its contiguous
shard of units and the only communication is an optional all-gather that reassembles the output on
every rank.  Kernels read local HBM only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


def shard_range(units: int, world_size: int, rank: int, granule: int = 1) -> Tuple[int, int]:
    """Contiguous ``[lo, hi)`` of ``units`` owned by ``rank``; shard boundaries are multiples of
    ``granule`` (e.g. 4 floats = one 16-byte vector, or 128 GEMM rows) and the tail goes to the last
    non-empty rank.  Ranks past the end get an empty range."""
    if units < 0 or world_size <= 0 or not 0 <= rank < world_size or granule <= 0:
        raise ValueError(f"bad shard request: units={units} world_size={world_size} rank={rank} granule={granule}")
    granules = -(-units // granule)
    per = -(-granules // world_size)
    lo = min(units, rank * per * granule)
    hi = min(units, (rank + 1) * per * granule)
    return lo, hi


def all_shard_ranges(units: int, world_size: int, granule: int = 1) -> List[Tuple[int, int]]:
    return [shard_range(units, world_size, r, granule) for r in range(world_size)]


@dataclass(frozen=True)
class Partition:
    """How one workload shards: the unit axis, its length and the replicated operands."""
    workload: str
    axis: str
    units: int
    granule: int
    replicated: Tuple[str, ...] = ()


def partition_for(workload: str, **dims: int) -> Partition:
    if workload == "vadd":
        return Partition(workload, "elements", dims["n"], 4)
    if workload == "softmax":
        return Partition(workload, "rows", dims["rows"], 1)
    if workload == "gemm_f16":
        return Partition(workload, "rows of A and C", dims["m"], 128, ("B", ))
    if workload == "gemm_i8":
        return Partition(workload, "rows of A and C", dims["m"], 128, ("B", "b_scale"))
    if workload == "attention":
        return Partition(workload, "batch x heads", dims["batch"] * dims["heads"], 1)
    raise ValueError(f"unknown workload {workload}")


def all_gather_units(local: torch.Tensor, units: int, world_size: int, granule: int = 1,
                     group: Optional["torch.distributed.ProcessGroup"] = None) -> torch.Tensor:
    """Reassemble the full output along dim 0 from every rank's shard (``local`` = this rank's
    ``[hi - lo, ...]`` slice).  Shards may be ragged; each is padded to the largest for the
    collective and trimmed afterwards."""
    import torch.distributed as dist
    ranges = all_shard_ranges(units, world_size, granule)
    rank = dist.get_rank(group)
    lo, hi = ranges[rank]
    if local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds {local.shape[0]} units, expected {hi - lo}")
    biggest = max(h - l for l, h in ranges)
    tail = tuple(local.shape[1:])
    if all(h - l == biggest for l, h in ranges):
        out = torch.empty((units, ) + tail, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest, ) + tail, dtype=local.dtype, device=local.device)
    padded[:hi - lo] = local
    pieces = [torch.empty_like(padded) for _ in range(world_size)]
    dist.all_gather(pieces, padded, group=group)
    return torch.cat([p[:h - l] for p, (l, h) in zip(pieces, ranges)], dim=0)
