"""``if`` on a run-time scalar (the block index, a loop variable) on CPU: the kernel is traced once per path and
every effect happens only for the blocks and iterations its conditions select (the reference emits ``scf.if``,
python/asc/codegen/function_visitor.py:585-627).  ``DRY_RUN=1`` stops before the device launch."""
import pytest
import torch

import asc
import asc2

N = 64


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


@asc2.jit
def even_odd(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int], tiles: int):
    x_gm, out_gm = asc2.tensor(x_ptr, [tiles * n]), asc2.tensor(out_ptr, [tiles * n])
    for t in range(asc2.block_idx(), tiles, asc2.block_num()):
        x = asc2.load(x_gm, [n], offsets=[t * n])
        if t % 2 == 0:
            asc2.store(x * 2, out_gm, offsets=[t * n])
        else:
            asc2.store(x + 1, out_gm, offsets=[t * n])


def test_branch_on_a_loop_variable_splits_the_iterations():
    x = torch.zeros(8 * N)
    even_odd[3](x, torch.zeros_like(x), N, 8)
    plan = even_odd.last_plan
    assert plan.pattern == "elementwise:program+elementwise:program"
    notes = [s.note for s in plan.steps]
    assert notes[:4] == [f"2 ops over [{t * N}, {(t + 1) * N})" for t in (0, 2, 4, 6)]       # the `then` arm: even tiles
    assert notes[4:] == [f"2 ops over [{t * N}, {(t + 1) * N})" for t in (1, 3, 5, 7)]       # the `else` arm: odd tiles
    assert plan.writes == {1} and plan.partial_writes == {1}


@asc2.jit
def first_blocks_only(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int], active: int):
    x_gm, out_gm = asc2.tensor(x_ptr, [8 * n]), asc2.tensor(out_ptr, [8 * n])
    b = asc2.block_idx()
    x = asc2.load(x_gm, [n], offsets=[b * n])
    if b < active:
        if b == 0:
            asc2.store(x - 1, out_gm, offsets=[0])
        else:
            asc2.store(asc2.exp(x), out_gm, offsets=[b * n])
    asc2.store(x, out_gm, offsets=[(b + 4) * n])          # after the join: every block


def test_nested_branches_on_the_block_index():
    x = torch.zeros(8 * N)
    first_blocks_only[4](x, torch.zeros_like(x), N, 3)
    notes = sorted(s.note for s in first_blocks_only.last_plan.steps)
    assert notes == sorted([
        f"2 ops over [1, {N}] pitches [{N}, {N}] from [0] to 0",             # block 0: x - 1 (stored at a fixed place)
        f"2 ops over [{N}, {3 * N})",                                         # blocks 1 and 2: exp(x), merged
        # the copy after the join is traced on all three paths; the three recordings are one computation under
        # complementary conditions and merge into one effect for all four blocks
        f"1 ops over [4, {N}] pitches [{N}, {N}] from [0] to {4 * N}",
    ])


@asc2.jit
def branch_on_data(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    x_gm, out_gm = asc2.tensor(x_ptr, [n]), asc2.tensor(out_ptr, [n])
    x = asc2.load(x_gm, [n], offsets=[0])
    if asc2.reduce_max(x) > 0:
        asc2.store(x, out_gm, offsets=[0])


def test_branch_on_tile_data_is_refused():
    with pytest.raises(NotImplementedError, match="not a function of the block index"):
        branch_on_data[1](torch.zeros(N), torch.zeros(N), N)


@asc2.jit
def branch_in_every_iteration(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    x_gm, out_gm = asc2.tensor(x_ptr, [8 * n]), asc2.tensor(out_ptr, [8 * n])
    for t in range(8):
        x = asc2.load(x_gm, [n], offsets=[t * n])
        if t < 3:
            x = x + 1
        if t % 4 == 0:
            x = x * 2
        asc2.store(x, out_gm, offsets=[t * n])


def test_two_branches_in_a_loop_give_four_guarded_stores():
    x = torch.zeros(8 * N)
    branch_in_every_iteration[1](x, torch.zeros_like(x), N)
    plan = branch_in_every_iteration.last_plan
    notes = sorted(s.note for s in plan.steps)
    # t < 3 and t % 4 == 0: t = 0; t < 3 only: t = 1, 2; t % 4 == 0 only: t = 4; neither: 3, 5, 6, 7
    assert notes == sorted([f"3 ops over [0, {N})", f"2 ops over [{N}, {3 * N})", f"2 ops over [{4 * N}, {5 * N})",
                            f"1 ops over [{3 * N}, {4 * N})", f"1 ops over [{5 * N}, {8 * N})"])


def test_compile_time_conditions_do_not_fork(monkeypatch):
    from asc.codegen import tracer
    runs = []
    real = tracer.TraceContext

    class Counting(real):
        def __init__(self, *a, **k):
            runs.append(1)
            super().__init__(*a, **k)
    monkeypatch.setattr(tracer, "TraceContext", Counting)

    @asc2.jit
    def static_if(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int], flag: asc.ConstExpr[bool],
                  count: int):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        if flag:
            x = x + 1
        if count > 2:              # a launch argument: known while tracing
            x = x * 2
        asc2.store(x, asc2.tensor(out_ptr, [n]), offsets=[0])
    static_if[1](torch.zeros(N), torch.zeros(N), N, True, 5)
    assert len(runs) == 1
    assert static_if.last_plan.steps[0].note.startswith("3 ops")


def test_too_many_paths_are_refused():
    @asc2.jit
    def seven_branches(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        b = asc2.block_idx()
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        for k in asc.static_range(7):
            if (b // (2 ** k)) % 2 == 1:
                x = x + 1
        asc2.store(x, asc2.tensor(out_ptr, [128 * n]), offsets=[b * n])
    with pytest.raises(NotImplementedError, match="more than 64 paths"):
        seven_branches[128](torch.zeros(N), torch.zeros(128 * N), N)


def test_a_while_loop_on_a_run_time_value_is_refused_instead_of_tracing_forever(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")

    @asc2.jit
    def while_loop(x_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress, n: int, tile: asc.ConstExpr[int]):
        x_gm, o_gm = asc2.tensor(x_ptr, [n]), asc2.tensor(o_ptr, [n])
        i = asc2.block_idx() * tile
        while i < n:
            asc2.store(asc2.load(x_gm, [tile], offsets=[i]) * 3.0, o_gm, offsets=[i])
            i += asc2.block_num() * tile

    with pytest.raises(NotImplementedError, match="while"):
        while_loop[4](torch.zeros(4096), torch.zeros(4096), 4096, 256)
