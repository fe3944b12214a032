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
from typing import Callable, List, Optional, Tuple

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


def rotated_shards(units: int, world_size: int, rank: int, granule: int = 1) -> List[Tuple[int, int]]:
    """The shards ``rank`` works on in consecutive passes over a fixed problem: its own in pass 0, then its
    neighbours' in turn.  In every pass the ranks together cover each shard exactly once (pass i: rank r takes
    shard (r + i) mod world_size), and no rank touches the same data in two consecutive passes, so a benchmark
    that repeats the problem never finds its inputs still in the GPU's L2."""
    ranges = all_shard_ranges(units, world_size, granule)
    return [ranges[(rank + i) % world_size] for i in range(world_size)]


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


def all_gather_in_place(full: torch.Tensor, units: int, world_size: int, granule: int = 1,
                        group: Optional["torch.distributed.ProcessGroup"] = None) -> None:
    """Reassemble the output where it lies: ``full`` is the whole, contiguous output (``units`` along dim 0 after
    flattening: ``full.numel() % units == 0``) in which this rank has written its own shard at the shard's place;
    on return every rank holds all of it.  Equal shards are one collective straight into ``full`` (no staging
    copy); ragged shards go through :func:`all_gather_units`."""
    import torch.distributed as dist
    if not full.is_contiguous() or units <= 0 or full.numel() % units:
        raise ValueError(f"output of {full.numel()} elements is not a contiguous array of {units} units")
    flat = full.view(-1)
    per_unit = flat.numel() // units
    ranges = all_shard_ranges(units, world_size, granule)
    lo, hi = ranges[dist.get_rank(group)]
    if len({h - l for l, h in ranges}) == 1:
        dist.all_gather_into_tensor(flat, flat[lo * per_unit:hi * per_unit], group=group)
        return
    local = flat[lo * per_unit:hi * per_unit].reshape(hi - lo, per_unit).clone()
    flat.copy_(all_gather_units(local, units, world_size, granule, group).view(-1))


def cyclic_chunks(units_per_rank: int, n_chunks: int) -> List[Tuple[int, int]]:
    """Local ``[lo, hi)`` pieces a rank's shard is produced in (equal on every rank)."""
    if units_per_rank < 0 or n_chunks <= 0:
        raise ValueError("bad chunking request")
    step = -(-max(units_per_rank, 1) // min(n_chunks, max(1, units_per_rank)))
    return [(lo, min(units_per_rank, lo + step)) for lo in range(0, units_per_rank, step)]


def cyclic_global_range(lo: int, hi: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Where local units ``[lo, hi)`` of ``rank`` sit in the gathered output: piece by piece the ranks'
    contributions lie side by side (a block-cyclic distribution), so each piece of every rank lands in one
    contiguous range that a single all-gather fills."""
    return world_size * lo + rank * (hi - lo), world_size * lo + (rank + 1) * (hi - lo)


def compute_and_gather(compute: Callable[[int, int], None], local: torch.Tensor, full: torch.Tensor, world_size: int,
                       n_chunks: int, group: Optional["torch.distributed.ProcessGroup"] = None) -> None:
    """Overlap the output all-gather with the computation that produces it.

    Every rank produces an equally sized shard ``local`` (``[units_per_rank, ...]``, a buffer ``compute``
    fills) in ``n_chunks`` pieces: ``compute(lo, hi)`` enqueues the kernel for local units ``[lo, hi)`` on the
    current stream, and as soon as a piece is enqueued its all-gather is started asynchronously, so the
    collective of piece i runs while piece i + 1 is computed.  Units are independent, so the gathered
    ``full`` (``[world_size * units_per_rank, ...]``) is laid out block-cyclically: piece by piece, rank after
    rank (``cyclic_global_range``); that keeps every collective a plain contiguous all-gather.  Returns when
    all of ``full`` is in place."""
    import torch.distributed as dist
    per = local.shape[0]
    if full.shape[0] != per * world_size or tuple(full.shape[1:]) != tuple(local.shape[1:]):
        raise ValueError(f"full output {tuple(full.shape)} is not {world_size} shards of {tuple(local.shape)}")
    works = []
    for lo, hi in cyclic_chunks(per, n_chunks):
        compute(lo, hi)
        works.append(dist.all_gather_into_tensor(full[world_size * lo:world_size * hi], local[lo:hi], group=group,
                                                 async_op=True))
    for w in works:
        w.wait()
