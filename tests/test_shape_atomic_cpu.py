"""Shape operations, broadcasts and atomics on CPU: the calls the launcher plans for the reference's
operation tests (python/test/asc2/operations/test_shape_ops.py, test_atomic_ops.py).  ``DRY_RUN=1`` stops
before the device launch."""
import pytest
import torch

import asc
import asc2

import asc2_scripts as K
import eltwise_cases as C


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


@pytest.mark.parametrize("asc_op, torch_op, args, shape, dtype", C.SHAPE_CASES, ids=C.ids)
def test_shape_op_plans(asc_op, torch_op, args, shape, dtype):
    launch, ref = C.shape_case(asc_op, torch_op, args, shape, dtype)
    launch()
    plan = K.shape_op.last_plan
    assert plan.pattern == "elementwise:program" and len(plan.steps) == 1 and plan.reads == {0} and plan.writes == {1}
    if asc_op is asc2.broadcast_to:      # one source row (pitch 0) repeated over the rows of the result
        assert plan.steps[0].note == f"1 ops over [{args[0]}, 32] pitches [0, 32] from [0] to 0"
    else:                                # a reshape keeps the row-major order: a flat copy
        n = ref.numel()
        assert plan.steps[0].note == f"1 ops over [1, {n}] pitches [{n}, {n}] from [0] to 0"
    assert not plan.partial_writes       # the result tensor is written completely


def test_constant_broadcast_needs_no_input():
    out = torch.zeros(3, 32, dtype=torch.int16)
    K.broadcast_dup[1](out, (3, 32), [0, 0])
    plan = K.broadcast_dup.last_plan
    assert plan.reads == set() and plan.writes == {0} and plan.steps[0].note.startswith("1 ops over [1, 96]")


@pytest.mark.parametrize("asc_op, torch_op, dtype", C.ATOMIC_CASES, ids=C.ids)
def test_atomic_plans_apply_blocks_in_order(asc_op, torch_op, dtype):
    launch, _ = C.atomic_case(asc_op, torch_op, dtype)
    launch()
    plan = K.atomic_op.last_plan
    kind = asc_op.__name__.split("_")[1]
    assert plan.pattern == f"atomic:{kind}" and plan.reads == {0, 1} and plan.writes == {1}
    # operand 0 is the accumulated window itself (in place), operand 1 block i's tile of x
    assert [s.note.split(" from ")[1] for s in plan.steps] == [f"[0, {32 * i}] to 0" for i in range(4)]


def test_bias_row_broadcast_merges_row_tiles():
    x = torch.zeros(4096, 1024)
    K.add_row_bias[16](x, torch.zeros(1, 1024), torch.zeros_like(x), 4096, 1024, 8)
    plan = K.add_row_bias.last_plan
    assert [s.note for s in plan.steps] == ["4 ops over [4096, 1024] pitches [1024, 0, 1024] from [0, 0] to 0"]
    assert plan.reads == {0, 1} and plan.writes == {2} and not plan.partial_writes


def test_concat_store_unfolds_into_one_store_per_part():
    a, b = torch.zeros(32, 64), torch.zeros(32, 64)
    K.concat_rows[4](a, b, torch.zeros(64, 64), 32, 32, 64, 8)
    plan = K.concat_rows.last_plan
    assert plan.reads == {0, 1} and plan.writes == {2} and plan.partial_writes == {2}
    assert len(plan.steps) == 8 and {s.fn_name for s in plan.steps} <= {"asc_cuda_eltwise_program",
                                                                         "asc_cuda_eltwise_program_2d"}
    K.concat_1d[1](torch.zeros(64), torch.zeros(64), torch.zeros(192), 64)
    assert len(K.concat_1d.last_plan.steps) == 3
    with pytest.raises(RuntimeError, match="same shape except their first dimension"):
        @asc2.jit
        def bad(x_ptr: asc.GlobalAddress):
            x_gm = asc2.tensor(x_ptr, [8, 16])
            asc2.concat(asc2.load(x_gm, [4, 16], offsets=[0, 0]), asc2.load(x_gm, [4, 8], offsets=[0, 0]))
        bad[1](torch.zeros(8, 16))
