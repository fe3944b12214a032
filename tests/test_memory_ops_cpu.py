"""Tile loads and stores anywhere in a tensor, on CPU: the windows the launcher plans for the reference's
memory-operation tests (python/test/asc2/operations/test_memory_ops.py).  ``DRY_RUN=1`` stops before the
device launch."""
import numpy as np
import pytest
import torch

import asc
import asc2

import asc2_scripts as K
import eltwise_cases as C


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


@pytest.mark.parametrize("case", C.MEMORY_CASES, ids=str)
def test_planned_window_is_the_addressed_tile(case):
    dim, tensor_shape, tile_shape, tile_id, offsets, _ = case
    launch, _, kernel = C.memory_case(*case)
    launch()
    plan = kernel.last_plan
    assert len(plan.steps) == 1 and plan.reads == {0, 1} and plan.writes == {2} and plan.partial_writes == {2}
    origin = [i * s for i, s in zip(tile_id, tile_shape)] if tile_id is not None else offsets
    note = plan.steps[0].note
    if tile_shape is None:                              # one element at the flat position
        flat = int(np.ravel_multi_index(origin, tensor_shape))
        assert note == f"3 ops over [{flat}, {flat + 1})"
    elif dim == 1:                                      # a clipped range
        lo, hi = origin[0], min(origin[0] + tile_shape[0], tensor_shape[0])
        assert note in (f"[{lo}, {hi})", f"3 ops over [{lo}, {hi})")
    elif tile_shape[1] == tensor_shape[1]:              # whole rows: a flat range
        lo = origin[0] * tensor_shape[1]
        assert note in (f"[{lo}, {lo + tile_shape[0] * tile_shape[1]})",
                        f"3 ops over [{lo}, {lo + tile_shape[0] * tile_shape[1]})")
    else:                                               # a strided 2-D window, clipped to the tensor
        rows = min(tile_shape[0], tensor_shape[0] - origin[0])
        cols = min(tile_shape[1], tensor_shape[1] - origin[1])
        assert note == f"3 ops over [{rows}, {cols}] at ({origin[0]}, {origin[1]})"


def test_tile_grid_of_all_blocks_collapses_into_one_flat_call():
    x = torch.zeros(1000, 1000)
    K.scale_2d_tiles[16](x, torch.zeros_like(x), 1000, 1000, 0.5, 64, 128)
    plan = K.scale_2d_tiles.last_plan
    assert [s.note for s in plan.steps] == ["3 ops over [0, 1000000)"]      # LOAD, MUL|IMM, TANH and not plan.partial_writes
    assert plan.pipeline is not None
    # with one tile left out the rest stays a list of windows and the output counts as partially written
    @asc2.jit
    def skip_first(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x_gm, out_gm = asc2.tensor(x_ptr, [n, n]), asc2.tensor(out_ptr, [n, n])
        for t in range(1 + asc2.block_idx(), 4, asc2.block_num()):
            asc2.store(asc2.exp(asc2.load(x_gm, [n // 2, n // 2], tile_id=[t // 2, t % 2])), out_gm,
                       tile_id=[t // 2, t % 2])
    y = torch.zeros(64, 64)
    skip_first[2](y, torch.zeros_like(y), 64)
    plan = skip_first.last_plan
    assert sorted(s.note for s in plan.steps) == ["2 ops over [32, 32] at (0, 32)", "2 ops over [32, 32] at (32, 0)",
                                                  "2 ops over [32, 32] at (32, 32)"]
    assert plan.partial_writes == {1}
