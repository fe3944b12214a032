"""Multi-GPU plumbing on CPU: shard arithmetic and the output all-gather over gloo, world size 2."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pyasc_b200 import sharding


def test_shard_ranges_cover_and_align():
    for units, world, gran in [(1 << 28, 8, 4), (16384, 8, 1), (8192, 8, 128), (128, 8, 1), (1000, 3, 4), (5, 8, 1),
                               (0, 2, 1), (130, 4, 128)]:
        ranges = sharding.all_shard_ranges(units, world, gran)
        assert ranges[0][0] == 0 and ranges[-1][1] == units
        for (l0, h0), (l1, h1) in zip(ranges, ranges[1:]):
            assert h0 == l1 and l0 <= h0
        for lo, hi in ranges:
            assert lo % gran == 0 or lo == units
    assert sharding.shard_range(8192, 8, 3, 128) == (3072, 4096)
    with pytest.raises(ValueError):
        sharding.shard_range(10, 2, 2)


def test_rotated_shards_cover_the_problem_once_per_pass():
    for units, world, gran in [(16384, 8, 1), (1 << 28, 4, 1 << 16), (8192, 2, 256), (128, 8, 1), (1000, 3, 4), (7, 1, 1)]:
        per_rank = [sharding.rotated_shards(units, world, r, gran) for r in range(world)]
        assert all(per_rank[r][0] == sharding.shard_range(units, world, r, gran) for r in range(world))
        for step in range(world):
            taken = sorted(per_rank[r][step] for r in range(world))
            assert taken == sharding.all_shard_ranges(units, world, gran)          # each shard exactly once
        if world > 1:
            assert all(per_rank[r][i] != per_rank[r][(i + 1) % world] for r in range(world) for i in range(world))


def test_partitions_name_the_replicated_operands():
    assert sharding.partition_for("gemm_f16", m=8192).replicated == ("B", )
    assert sharding.partition_for("gemm_i8", m=8192).replicated == ("B", "b_scale")
    assert sharding.partition_for("attention", batch=4, heads=32).units == 128
    assert sharding.partition_for("vadd", n=1 << 28).granule == 4


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, units: int, gran: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(units * 3, dtype=torch.float32).reshape(units, 3)
        lo, hi = sharding.shard_range(units, world, rank, gran)
        # each rank "computes" only its shard (here: x + 1) and the gather reassembles the whole output
        local = full[lo:hi] + 1
        out = sharding.all_gather_units(local, units, world, gran)
        assert torch.equal(out, full + 1), f"rank {rank}"
        with pytest.raises(ValueError):
            sharding.all_gather_units(local[:-1] if hi > lo else torch.zeros(1, 3), units, world, gran)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("units, gran", [(64, 1), (1000, 4), (130, 128)])
def test_all_gather_over_gloo(units, gran):
    mp.spawn(_worker, args=(2, _free_port(), units, gran), nprocs=2, join=True)


def _in_place_worker(rank: int, world: int, port: int, units: int, gran: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        want = torch.arange(units * 5, dtype=torch.float32).reshape(units, 5) * 3
        full = torch.full((units, 5), -1.0)
        lo, hi = sharding.shard_range(units, world, rank, gran)
        full[lo:hi] = want[lo:hi]                      # this rank's shard, written at its place
        sharding.all_gather_in_place(full, units, world, gran)
        assert torch.equal(full, want), f"rank {rank}"
        with pytest.raises(ValueError):
            sharding.all_gather_in_place(full[:, :3], units, world, gran)      # not contiguous
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("units, gran", [(64, 1), (1024, 256), (1000, 4), (130, 128)])
def test_all_gather_in_place_over_gloo(units, gran):
    mp.spawn(_in_place_worker, args=(2, _free_port(), units, gran), nprocs=2, join=True)


def _overlap_worker(rank: int, world: int, port: int, per: int, chunks: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # global unit g holds the value g; every rank "computes" (x * 2) the units the cyclic layout gives it
        local = torch.zeros(per, 2)
        full = torch.full((world * per, 2), -1.0)
        calls = []

        def compute(lo, hi):
            calls.append((lo, hi))
            g0, g1 = sharding.cyclic_global_range(lo, hi, rank, world)
            local[lo:hi] = torch.arange(g0, g1, dtype=torch.float32)[:, None].expand(-1, 2) * 2

        sharding.compute_and_gather(compute, local, full, world, chunks)
        want = torch.arange(world * per, dtype=torch.float32)[:, None].expand(-1, 2) * 2
        assert torch.equal(full, want), f"rank {rank}"
        assert calls == sharding.cyclic_chunks(per, chunks)
        assert calls[0][0] == 0 and calls[-1][1] == per and all(a[1] == b[0] for a, b in zip(calls, calls[1:]))
        with pytest.raises(ValueError):
            sharding.compute_and_gather(compute, local, full[:-1], world, chunks)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("per, chunks", [(64, 4), (10, 3), (5, 8)])
def test_compute_and_gather_overlapped_over_gloo(per, chunks):
    mp.spawn(_overlap_worker, args=(2, _free_port(), per, chunks), nprocs=2, join=True)


def test_cyclic_layout_covers_every_unit_once():
    for per, chunks, world in [(64, 4, 2), (10, 3, 4), (5, 8, 8), (1, 1, 3)]:
        seen = []
        for r in range(world):
            for lo, hi in sharding.cyclic_chunks(per, chunks):
                g0, g1 = sharding.cyclic_global_range(lo, hi, r, world)
                seen += list(range(g0, g1))
        assert sorted(seen) == list(range(per * world))
