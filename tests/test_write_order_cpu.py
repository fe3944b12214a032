"""Stores that overlap in the output, on CPU: a plan must leave the data the kernel's own order leaves
(within a block: iteration after iteration, store after store), or refuse the kernel.  ``DRY_RUN=1`` stops
before the device launch."""
import pytest
import torch

import asc
import asc2
from asc.codegen.matcher import UnsupportedKernelError


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


N = 64


@asc2.jit
def every_iteration_stores_to_the_front(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    x_gm, y_gm = asc2.tensor(x_ptr, [4 * n]), asc2.tensor(y_ptr, [4 * n])
    for i in range(4):
        asc2.store(asc2.load(x_gm, [n], offsets=[i * n]) + 1, y_gm, offsets=[0])


def test_last_iteration_wins_when_all_write_one_window():
    x = torch.zeros(4 * N)
    every_iteration_stores_to_the_front[1](x, torch.zeros_like(x), N)
    plan = every_iteration_stores_to_the_front.last_plan
    # one call per iteration, in iteration order: the tile loaded at 3 n is written last
    assert [s.note.split(" from ")[1] for s in plan.steps] == [f"[{i * N}] to 0" for i in range(4)]


@asc2.jit
def descending_half_overlaps(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    x_gm, y_gm = asc2.tensor(x_ptr, [4 * n]), asc2.tensor(y_ptr, [4 * n])
    for i in range(4):
        asc2.store(asc2.load(x_gm, [n], offsets=[i * n]) * 2, y_gm, offsets=[(3 - i) * (n // 2)])


def test_half_overlapping_windows_keep_iteration_order():
    x = torch.zeros(4 * N)
    descending_half_overlaps[1](x, torch.zeros_like(x), N)
    plan = descending_half_overlaps.last_plan
    assert [s.note.split(" from ")[1] for s in plan.steps] == [f"[{i * N}] to {(3 - i) * (N // 2)}" for i in range(4)]


@asc2.jit
def disjoint_windows_from_other_positions(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    x_gm, y_gm = asc2.tensor(x_ptr, [4 * n]), asc2.tensor(y_ptr, [4 * n])
    for i in range(asc2.block_idx(), 4, asc2.block_num()):
        asc2.store(asc2.load(x_gm, [n], offsets=[(3 - i) * n]) * 2, y_gm, offsets=[i * n])


def test_disjoint_windows_are_still_sorted_and_repeat_free():
    x = torch.zeros(4 * N)
    disjoint_windows_from_other_positions[2](x, torch.zeros_like(x), N)
    plan = disjoint_windows_from_other_positions.last_plan
    assert [s.note.split(" from ")[1] for s in plan.steps] == [f"[{(3 - i) * N}] to {i * N}" for i in range(4)]


@asc2.jit
def second_store_runs_ahead(a_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    a_gm, y_gm = asc2.tensor(a_ptr, [n]), asc2.tensor(y_ptr, [5 * n])
    a = asc2.load(a_gm, [n], offsets=[0])
    for i in range(4):
        asc2.store(a + 1, y_gm, offsets=[i * n])
        asc2.store(a * 2, y_gm, offsets=[(i + 1) * n])


def test_store_overwritten_by_a_later_iteration_of_an_earlier_store_is_refused():
    # iteration i + 1 overwrites with `a + 1` what iteration i stored as `a * 2`; "all of the first store, then all
    # of the second" would leave `a * 2` in y[n : 4 n]
    with pytest.raises(UnsupportedKernelError, match="later loop iteration"):
        second_store_runs_ahead[1](torch.zeros(N), torch.zeros(5 * N), N)


@asc2.jit
def second_store_in_step(a_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    a_gm, y_gm = asc2.tensor(a_ptr, [n]), asc2.tensor(y_ptr, [8 * n])
    a = asc2.load(a_gm, [n], offsets=[0])
    for i in range(4):
        asc2.store(a + 1, y_gm, offsets=[2 * i * n])
        asc2.store(a * 2, y_gm, offsets=[2 * i * n + n // 2])      # overlaps the first store of the same iteration only


def test_overlap_inside_one_iteration_keeps_program_order():
    second_store_in_step[1](torch.zeros(N), torch.zeros(8 * N), N)
    plan = second_store_in_step.last_plan
    assert plan.pattern == "elementwise:program+elementwise:program" and len(plan.steps) == 8


@asc2.jit
def reduce_into_one_slot(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: asc.ConstExpr[int],
                         cols: asc.ConstExpr[int]):
    x_gm, out_gm = asc2.tensor(x_ptr, [4 * rows, cols]), asc2.tensor(out_ptr, [4 * rows])
    for i in range(4):
        tile = asc2.load(x_gm, [rows, cols], offsets=[i * rows, 0])
        asc2.store(asc2.reduce_sum(tile, 1), out_gm, offsets=[0])


def test_reductions_of_different_tiles_into_one_range_are_refused():
    with pytest.raises(UnsupportedKernelError, match="overlapping ranges"):
        reduce_into_one_slot[1](torch.zeros(32, 64), torch.zeros(32), 8, 64)
