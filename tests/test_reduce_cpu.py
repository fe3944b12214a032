"""Reduction and softmax-op kernels on CPU: the plans the launcher builds for the reference's operation
tests (python/test/asc2/operations/test_reduce_ops.py, test_softmax.py).  ``DRY_RUN=1`` stops before
the device launch."""
import pytest
import torch

import asc
import asc2

import asc2_scripts as K


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


def step_of(jit_fn):
    plan = jit_fn.last_plan
    assert len(plan.steps) == 1, plan
    return plan, plan.steps[0]


@pytest.mark.parametrize("dim, keep_dims, note", [
    (0, False, "axis 0 of [64, 32] at (0, 0) -> [0, +32)"),
    (1, False, "axis 1 of [64, 32] at (0, 0) -> [0, +64)"),
    (0, True, "axis 0 of [64, 32] at (0, 0) -> [0, +32)"),
])
def test_axis_reduction_plans(dim, keep_dims, note):
    x = torch.zeros(64, 32)
    out_shape = [64, 32]
    if keep_dims:
        out_shape[dim] = 1
    else:
        del out_shape[dim]
    K.reduce_axis[1](x, torch.zeros(out_shape), dim, [64, 32], [0, 0], out_shape, [0] * len(out_shape), asc2.reduce_min,
                     keep_dims)
    plan, step = step_of(K.reduce_axis)
    assert plan.pattern == "reduce:min" and step.fn_name == "asc_cuda_reduce_f32" and step.note == "min " + note
    assert plan.reads == {0} and plan.writes == {1} and not plan.partial_writes


def test_full_reduction_fills_the_stored_tile():
    x = torch.zeros(64, 32)
    K.reduce_all[1](x, torch.zeros(32), [64, 32], [0, 0], [32], [0], asc2.reduce_sum)
    assert step_of(K.reduce_all)[1].note == "sum axis -1 of [64, 32] at (0, 0) -> [0, +32)"
    for tile in (1, 7, 17):
        K.reduce_tile[1](torch.zeros(32), torch.empty(1), 32, tile_size=tile)
        assert step_of(K.reduce_tile)[1].note == f"max axis -1 of [1, {tile}] at (0, 0) -> [0, +1)"


def test_row_tiles_of_all_blocks_merge_into_one_call():
    x = torch.zeros(4096, 1024)
    K.row_sums[16](x, torch.empty(4096), 4096, 1024, 8)
    plan, step = step_of(K.row_sums)
    assert step.note == "sum axis 1 of [4096, 1024] at (0, 0) -> [0, +4096)" and not plan.partial_writes
    # keep_dims along the last axis would make a [rows, 1] tile, which the surface rejects like the reference
    with pytest.raises(RuntimeError, match="aligned by 32 bytes"):
        K.reduce_axis[1](x, torch.zeros(4096, 1), 1, [4096, 1024], [0, 0], [4096, 1], [0, 0], asc2.reduce_sum, True)


def test_reduction_rejections():
    x = torch.zeros(64, 32)
    with pytest.raises(NotImplementedError, match="past the end"):
        K.reduce_axis[1](x, torch.zeros(32), 0, [64, 32], [32, 0], [32], [0], asc2.reduce_sum, False)
    # fp16 tiles reduced along the first axis take the column program (fp32 combination, one rounding) ...
    K.reduce_axis[1](x.half(), torch.zeros(32, dtype=torch.float16), 0, [64, 32], [0, 0], [32], [0], asc2.reduce_sum,
                     False)
    assert step_of(K.reduce_axis)[0].pattern == "reduce:sum:columns"
    # ... a whole fp16 tile has the 16-bit form of the whole-window kernel ...
    K.reduce_all[1](x.half(), torch.zeros(32, dtype=torch.float16), [64, 32], [0, 0], [32], [0], asc2.reduce_max)
    assert step_of(K.reduce_all)[1].fn_name == "asc_cuda_reduce_all_f16"
    # ... integer tiles have no reduction kernel (nor has the reference: Ascend C reduces half and float)
    with pytest.raises(NotImplementedError, match="float32 only"):
        K.reduce_axis[1](x.int(), torch.zeros(32, dtype=torch.int32), 0, [64, 32], [0, 0], [32], [0], asc2.reduce_sum,
                         False)


def test_softmax_op_plans_and_identity_store():
    s = torch.zeros(4, 256)
    K.softmax_2d[1](torch.zeros_like(s), s, [4, 256])
    plan, step = step_of(K.softmax_2d)        # the store of the unchanged source tile adds no call
    assert step.fn_name == "asc_cuda_softmax_f32" and step.note == "rows [0, 4) x 256 cols"
    assert plan.reads == {1} and plan.writes == {0}
    v = torch.zeros(1024)
    K.softmax_1d[1](torch.zeros_like(v), v, 1024)
    assert step_of(K.softmax_1d)[1].note == "rows [0, 1) x 1024 cols"


def test_rms_norm_plans():
    """asc2.rms_norm over whole rows becomes one fused call per contiguous row range; gamma stays resident when
    the launcher streams the rows in chunks."""
    x = torch.zeros(4096, 1024)
    K.rms_norm_rows[16](x, torch.ones(1, 1024), torch.empty_like(x), 4096, 1024, 8, 1e-5)
    plan, step = step_of(K.rms_norm_rows)
    assert plan.pattern == "rms_norm" and step.fn_name == "asc_cuda_rms_norm_f32"
    assert step.note == "rows [0, 4096) x 1024 cols"
    assert plan.reads == {0, 1} and plan.writes == {2} and not plan.partial_writes
    assert plan.pipeline is not None and plan.pipeline.resident == {1} and plan.pipeline.units == 4096
    args = step.build({0: 1 << 20, 1: 2 << 20, 2: 3 << 20}, None)
    assert [a.value for a in args[:6]] == [1 << 20, 2 << 20, 3 << 20, 4096, 1024, 1024]
    assert args[6].value == pytest.approx(1e-5)
    # rows not all covered: a partial write, no pipelining
    K.rms_norm_rows[1](x, torch.ones(1, 1024), torch.empty_like(x), 4096, 1024, 8, 1e-5)
    assert K.rms_norm_rows.last_plan.steps[0].note == "rows [0, 4096) x 1024 cols"
    K.rms_norm_1d[1](torch.zeros(256), torch.ones(256), torch.empty(256), 256)
    assert step_of(K.rms_norm_1d)[1].note == "rows [0, 1) x 256 cols"
    with pytest.raises(RuntimeError, match="float32 and float16"):
        K.rms_norm_1d[1](torch.zeros(256, dtype=torch.int32), torch.ones(256, dtype=torch.int32),
                         torch.empty(256, dtype=torch.int32), 256)
    K.rms_norm_1d[1](torch.zeros(256, dtype=torch.float16), torch.ones(256, dtype=torch.float16),
                     torch.empty(256, dtype=torch.float16), 256)
    assert step_of(K.rms_norm_1d)[1].fn_name == "asc_cuda_rms_norm_f16"


def test_column_reduction_of_a_computed_tile_plans_one_column_program_per_tile(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")

    @asc2.jit
    def col_norms(x_ptr: asc.GlobalAddress, w_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, tiles: int,
                  rows: asc.ConstExpr[int], cols: asc.ConstExpr[int]):
        x_gm = asc2.tensor(x_ptr, [tiles * rows, cols])
        out_gm = asc2.tensor(out_ptr, [tiles, cols])
        w = asc2.load(asc2.tensor(w_ptr, [1, cols]), [1, cols], offsets=[0, 0])
        for t in range(asc2.block_idx(), tiles, asc2.block_num()):
            x = asc2.load(x_gm, [rows, cols], offsets=[t * rows, 0])
            y = x * w.broadcast_to(rows, cols)
            asc2.store(asc2.reduce_max(y * y, 0, keep_dims=True), out_gm, offsets=[t, 0])
    x = torch.zeros(6 * 32, 256)
    col_norms[4](x, torch.zeros(1, 256), torch.zeros(6, 256), 6, 32, 256)
    plan = col_norms.last_plan
    assert plan.pattern == "reduce:max:columns" and plan.reads == {0, 1} and plan.writes == {2}
    assert [s.note.split(" from ")[1] for s in plan.steps] == [f"[{t * 32 * 256}, 0] to {t * 256}" for t in range(6)]
    assert not plan.partial_writes                    # six rows of 256: the whole output


def test_half_precision_row_reductions_plan_as_row_programs(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")

    @asc2.jit
    def row_sums(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, cols: asc.ConstExpr[int],
                 rpt: asc.ConstExpr[int]):
        x_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(out_ptr, [rows])
        for i in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
            asc2.store(asc2.reduce_sum(asc2.load(x_gm, [rpt, cols], offsets=[i, 0]), 1), out_gm, offsets=[i])
    for dtype, round_op in ((torch.float16, 33), (torch.bfloat16, 34)):
        row_sums[4](torch.zeros(64, 512, dtype=dtype), torch.zeros(64, dtype=dtype), 64, 512, 8)
        (step, ) = row_sums.last_plan.steps
        built = step.build({0: 0, 1: 0}, None)
        assert list(built[0][:3]) == [0, 59, round_op]          # LOAD, ROW_SUM in fp32, one rounding to the tile type
