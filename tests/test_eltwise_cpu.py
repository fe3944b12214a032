"""Elementwise asc2 kernels on CPU: the launcher's compiled postfix program, evaluated by the CPU
oracle, must reproduce the torch goldens of the reference's tests
(python/test/asc2/operations/test_{binary_ops,unary_ops,where}.py,
python/test/asc2/kernels/test_{leaky_relu,gelu}.py).  ``DRY_RUN=1`` stops before the device launch."""
import numpy as np
import pytest
import torch

import asc
import asc2

import asc2_scripts as K
import eltwise_cases as C
from oracle import eltwise as E


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


def decode(step):
    """(ops, args, runtime-argument index of each input, output index, out_type, n) of a program step."""
    assert step.fn_name == "asc_cuda_eltwise_program"
    ptrs = {i: (i + 1) << 32 for i in range(16)}
    built = step.build(ptrs, None)
    ops, args, n_ops, ins, types, n_in, out, out_type, n, _ = built
    assert len(ops) == n_ops.value and len(ins) == n_in.value
    in_idx = [(int(a) >> 32) - 1 for a in ins]
    return list(ops), list(args), in_idx, list(types), (out.value >> 32) - 1, out_type.value, n.value


def evaluate(jit_fn, runtime_args):
    plan = jit_fn.last_plan
    if plan.pattern == "elementwise:asc_cuda_vadd_f32":   # fp32 tile + tile keeps its dedicated kernel
        assert plan.reads == {0, 1} and plan.writes == {2}
        return runtime_args[0] + runtime_args[1]
    assert plan.pattern == "elementwise:program" and len(plan.steps) == 1, plan
    ops, args, in_idx, types, out_idx, out_type, n = decode(plan.steps[0])
    inputs = [runtime_args[i].reshape(-1)[:n] for i in in_idx]
    assert [E.TYPES[t] for t in types] == [t.dtype for t in inputs]
    assert plan.reads == set(in_idx) and plan.writes == {out_idx}
    return E.run_program(ops, args, inputs, out_type).reshape(runtime_args[out_idx].shape)


def check(out, golden):
    assert out.dtype == golden.dtype
    if golden.dtype == torch.float32:
        assert torch.allclose(out, golden, atol=1e-3)
    else:
        assert torch.equal(out, golden)


@pytest.mark.parametrize("asc_op, torch_op, fmt, dtype", C.BINARY_CASES, ids=C.ids)
def test_binary_programs(asc_op, torch_op, fmt, dtype):
    launch, golden, rt_args = C.binary_case(asc_op, torch_op, fmt, dtype)
    launch()
    check(evaluate(K.binary_op, rt_args), golden)


@pytest.mark.parametrize("asc_op, torch_op", C.UNARY_OPS, ids=C.ids)
def test_unary_programs(asc_op, torch_op):
    launch, golden, rt_args = C.unary_case(asc_op, torch_op)
    launch()
    check(evaluate(K.unary_op, rt_args), golden)


@pytest.mark.parametrize("scalar", [False, True], ids=["tile", "scalar"])
@pytest.mark.parametrize("dtype", C.WHERE_DTYPES, ids=str)
@pytest.mark.parametrize("asc_op, torch_op", C.COMPARE_OPS, ids=C.ids)
def test_where_programs(asc_op, torch_op, dtype, scalar):
    launch, golden, rt_args = C.where_case(asc_op, torch_op, dtype, scalar)
    launch()
    out = evaluate(K.where_scalar_op if scalar else K.where_op, rt_args)
    assert torch.equal(out, golden)


def test_leaky_relu_program_is_exact_in_bf16():
    launch, golden, rt_args = C.leaky_relu_case()
    launch()
    plan = K.leaky_relu.last_plan
    # x >= 0 and x * alpha take their scalars as immediates: LOAD, LE|IMM, LOAD, LOAD, MUL|IMM, ROUND, WHERE
    assert plan.steps[0].note == "7 ops over [0, 8192)" and plan.pipeline is not None
    ops = decode(plan.steps[0])[0]
    assert ops == [0, 31 | 0x100, 0, 0, 4 | 0x100, 34, 32]
    assert torch.equal(evaluate(K.leaky_relu, rt_args), golden)


@pytest.mark.parametrize("approximate", [True, False])
def test_gelu_program(approximate):
    launch, golden, rt_args = C.gelu_case(approximate)
    launch()
    torch.testing.assert_close(evaluate(K.gelu, rt_args), golden, rtol=1e-3, atol=1e-5)
    # operand reordering keeps the whole expression within two stack levels
    ops = decode(K.gelu.last_plan.steps[0])[0]
    depth = peak = 0
    for op in ops:
        code, imm = op & 0xff, bool(op & 0x100)
        depth += 1 if code <= 1 else 0 if imm or code in range(8, 26) or code in (33, 34) else -1
        peak = max(peak, depth)
    assert depth == 1 and peak == 2 and len(ops) == (13 if approximate else 7)


def test_sixteen_bit_chain_rounds_after_every_op():
    @asc2.jit
    def chain(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        y = asc2.load(asc2.tensor(y_ptr, [n]), [n], offsets=[0])
        asc2.store(asc2.exp(x * y + 0.3) - y, asc2.tensor(out_ptr, [n]), offsets=[0])
    gen = torch.Generator().manual_seed(7)
    x = torch.rand(256, generator=gen).to(torch.float16)
    y = torch.rand(256, generator=gen).to(torch.float16)
    out = torch.empty_like(x)
    chain[1](x, y, out, 256)
    golden = torch.exp(x * y + torch.tensor(0.3, dtype=torch.float16)) - y     # every op rounds to fp16
    assert torch.equal(evaluate(chain, [x, y, out]), golden)


def test_cast_between_float_and_int():
    @asc2.jit
    def to_int(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        asc2.store((x * 3.5).to(asc.int32), asc2.tensor(out_ptr, [n]), offsets=[0])
    x = torch.linspace(-40, 40, 64)
    out = torch.empty(64, dtype=torch.int32)
    to_int[1](x, out, 64)
    assert torch.equal(evaluate(to_int, [x, out]), (x * 3.5).to(torch.int32))


def test_program_limits_and_rejections():
    @asc2.jit
    def deep(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        v = x
        for _ in asc.static_range(60):
            v = v * 1.5 + x
        asc2.store(v, asc2.tensor(out_ptr, [n]), offsets=[0])
    x = torch.zeros(64)
    with pytest.raises(NotImplementedError, match="limits"):
        deep[1](x, torch.empty_like(x), 64)

    @asc2.jit
    def in_place(x_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x_gm = asc2.tensor(x_ptr, [n])
        asc2.store(asc2.exp(asc2.load(x_gm, [n], offsets=[0])), x_gm, offsets=[0])
    with pytest.raises(NotImplementedError, match="also loads"):
        in_place[1](x, 64)

    @asc2.jit
    def shifted(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [2 * n]), [n], offsets=[n])
        asc2.store(asc2.exp(x), asc2.tensor(out_ptr, [2 * n]), offsets=[0])
    shifted[1](torch.zeros(128), torch.zeros(128), 64)       # operands addressed differently: one call per tile
    assert [st.note for st in shifted.last_plan.steps] == ["2 ops over [1, 64] pitches [64, 64] from [64] to 0"]
    with pytest.raises(NotImplementedError, match="also loads at other positions"):
        @asc2.jit
        def shift_in_place(x_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
            x_gm = asc2.tensor(x_ptr, [2 * n])
            asc2.store(asc2.exp(asc2.load(x_gm, [n], offsets=[n])), x_gm, offsets=[0])
        shift_in_place[1](torch.zeros(128), 64)


def test_golden_fixture_through_compiled_programs(golden_dir):
    """The committed fixture (tests/golden/make_golden.py) against the programs the launcher compiles,
    evaluated by the CPU oracle."""
    import os
    d = np.load(os.path.join(golden_dir, "elementwise_reduce.npz"))
    x = torch.from_numpy(d["gelu_x"])
    out = torch.empty_like(x)
    for approximate, key in ((False, "gelu_erf"), (True, "gelu_tanh")):
        K.gelu[16](x, out, 8, 1024, 1024, approximate)
        torch.testing.assert_close(evaluate(K.gelu, [x, out]), torch.from_numpy(d[key]), rtol=1e-3, atol=1e-5)
    xl = torch.from_numpy(d["leaky_x"]).view(torch.bfloat16)
    alpha = torch.tensor(float(d["leaky_alpha"]), dtype=torch.bfloat16)
    ol = torch.empty_like(xl)
    K.leaky_relu[16](xl, alpha, ol, 8192, 128, 4)
    assert torch.equal(evaluate(K.leaky_relu, [xl, alpha, ol, 8192]), torch.from_numpy(d["leaky_out"]).view(torch.bfloat16))


def test_sigmoid_and_silu_compile_to_the_specialised_programs():
    """The library has compile-time instances for exactly these opcode sequences."""
    @asc2.jit
    def sigmoid(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        asc2.store(1 / (1 + asc2.exp(-x)), asc2.tensor(out_ptr, [n]), offsets=[0])

    @asc2.jit
    def silu(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        asc2.store(x / (asc2.exp(-x) + 1), asc2.tensor(out_ptr, [n]), offsets=[0])
    x = torch.linspace(-6, 6, 256)
    out = torch.empty_like(x)
    sigmoid[1](x, out, 256)
    assert decode(sigmoid.last_plan.steps[0])[0] == [0, 8, 11, 2 | 0x100, 5 | 0x100]
    torch.testing.assert_close(evaluate(sigmoid, [x, out]), torch.sigmoid(x), rtol=1e-6, atol=1e-7)
    silu[1](x, out, 256)
    assert decode(silu.last_plan.steps[0])[0] == [0, 0, 8, 11, 2 | 0x100, 5]
    torch.testing.assert_close(evaluate(silu, [x, out]), torch.nn.functional.silu(x), rtol=1e-6, atol=1e-6)


def test_expression_graph_that_explodes_as_a_tree_is_refused_quickly():
    """y = y + y forty times: 2^40 leaves as a tree; the compiler must refuse it instead of unfolding it."""
    @asc2.jit
    def doubling(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        y = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        for _ in asc.static_range(40):
            y = y * 2 + y
        asc2.store(y, asc2.tensor(out_ptr, [n]), offsets=[0])
    with pytest.raises(NotImplementedError, match="unfolds into more than"):
        doubling[1](torch.zeros(64), torch.zeros(64), 64)


def test_tile_carried_across_loop_iterations_unrolls_the_loop():
    """A loop body is traced once, so a tile that one iteration hands to the next cannot be represented by that
    trace: the launcher traces again with the short compile-time loop unrolled and plans the data flow; a loop too
    long to unroll is refused instead of computing a single iteration."""
    @asc2.jit
    def running_sum(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int], reps: int):
        x_gm = asc2.tensor(x_ptr, [reps * n])
        acc = asc2.zeros([n], dtype=asc.float32)
        for i in range(reps):
            acc = acc + asc2.load(x_gm, [n], offsets=[i * n])
        asc2.store(acc, asc2.tensor(out_ptr, [n]), offsets=[0])
    running_sum[1](torch.zeros(256), torch.zeros(64), 64, 4)
    (step, ) = running_sum.last_plan.steps
    # 0 + x0 + x1 + x2 + x3: four loads from four places, four additions (the first with the constant 0)
    assert step.note == "8 ops over [1, 64] pitches [64, 64, 64, 64, 64] from [0, 64, 128, 192] to 0"
    with pytest.raises(NotImplementedError, match="carried across iterations"):
        running_sum[1](torch.zeros(6464), torch.zeros(64), 64, 101)


def test_tile_loaded_before_an_overwrite_of_its_tensor_is_refused():
    """Effects run one after the other over all blocks, so a tile loaded before a store to its tensor and used
    after it would see the new contents: the launcher must refuse; loading again after the store is fine."""
    @asc2.jit
    def stale(x_ptr: asc.GlobalAddress, z_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x_gm, z_gm, y_gm = (asc2.tensor(p, [n]) for p in (x_ptr, z_ptr, y_ptr))
        old = asc2.load(x_gm, [n], offsets=[0])
        asc2.store(asc2.load(z_gm, [n], offsets=[0]) * 2, x_gm, offsets=[0])
        asc2.store(old + 1, y_gm, offsets=[0])
    with pytest.raises(NotImplementedError, match="loaded before an earlier store"):
        stale[1](torch.zeros(64), torch.zeros(64), torch.zeros(64), 64)

    @asc2.jit
    def fresh(x_ptr: asc.GlobalAddress, z_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x_gm, z_gm, y_gm = (asc2.tensor(p, [n]) for p in (x_ptr, z_ptr, y_ptr))
        asc2.store(asc2.load(z_gm, [n], offsets=[0]) * 2, x_gm, offsets=[0])
        asc2.store(asc2.load(x_gm, [n], offsets=[0]) + 1, y_gm, offsets=[0])
    fresh[1](torch.zeros(64), torch.zeros(64), torch.zeros(64), 64)
    assert len(fresh.last_plan.steps) == 2


def test_reading_back_another_blocks_output_is_refused():
    @asc2.jit
    def neighbour(z_ptr: asc.GlobalAddress, x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int],
                  total: asc.ConstExpr[int]):
        z_gm, x_gm, y_gm = (asc2.tensor(p, [total]) for p in (z_ptr, x_ptr, y_ptr))
        i = asc2.block_idx() * n
        asc2.store(asc2.load(z_gm, [n], offsets=[i]) * 2, x_gm, offsets=[i])
        asc2.store(asc2.load(x_gm, [n], offsets=[0]) + 1, y_gm, offsets=[i])      # block 0's output, read by all
    with pytest.raises(NotImplementedError, match="reads a tensor back at other positions"):
        neighbour[4](torch.zeros(256), torch.zeros(256), torch.zeros(256), 64, 256)

    @asc2.jit
    def own(z_ptr: asc.GlobalAddress, x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, n: asc.ConstExpr[int],
            total: asc.ConstExpr[int]):
        z_gm, x_gm, y_gm = (asc2.tensor(p, [total]) for p in (z_ptr, x_ptr, y_ptr))
        i = asc2.block_idx() * n
        asc2.store(asc2.load(z_gm, [n], offsets=[i]) * 2, x_gm, offsets=[i])
        asc2.store(asc2.load(x_gm, [n], offsets=[i]) + 1, y_gm, offsets=[i])      # each block reads what it wrote
    own[4](torch.zeros(256), torch.zeros(256), torch.zeros(256), 64, 256)
    assert len(own.last_plan.steps) == 2


def test_count_mask_plans_one_call_per_tile_with_the_element_index(monkeypatch):
    """``with asc2.mask(count=n, other=v)``: the operations inside keep their first n elements and hold v in the
    rest, so the program compares the element index inside the tile with n; tiles are then planned one call each
    (the index restarts with every tile) instead of being merged into one flat range."""
    monkeypatch.setenv("DRY_RUN", "1")

    @asc2.jit
    def masked_scale(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int], count: int):
        x_gm, out_gm = asc2.tensor(x_ptr, [4 * n]), asc2.tensor(out_ptr, [4 * n])
        for t in range(asc2.block_idx(), 4, asc2.block_num()):
            x = asc2.load(x_gm, [n], offsets=[t * n])
            with asc2.mask(count=count, other=-1.0):
                y = x * 2
            asc2.store(y, out_gm, offsets=[t * n])
    masked_scale[2](torch.zeros(256), torch.zeros(256), 64, 10)
    plan = masked_scale.last_plan
    assert [s.note.split(" from ")[1] for s in plan.steps] == [f"[{t * 64}] to {t * 64}" for t in range(4)]
    ops = list(plan.steps[0].build({0: 0, 1: 0}, None)[0][:plan.steps[0].build({0: 0, 1: 0}, None)[2].value])
    assert 65 in ops and 32 in ops                           # INDEX ... WHERE
    with pytest.raises(NotImplementedError, match="bits"):
        @asc2.jit
        def bit_mask(x_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
            x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
            with asc2.mask(bits=(0, 255)):
                asc2.store(x + 1, asc2.tensor(x_ptr, [n]), offsets=[0])
        bit_mask[1](torch.zeros(64), 64)


def test_in_place_update_of_the_stored_window_plans_and_other_positions_are_refused():
    """`y = x + y` through scalar-sized tiles, as in the reference's loop-unrolling note
    (docs/design/software-pipelining.md:55-66): the operand taken from the stored tensor is the stored window
    itself, so each element is read by the thread that overwrites it.  Shifted by one element it is refused."""
    @asc2.jit()
    def accumulate(x, y, size: int):
        x_gm = asc2.tensor(x, [size])
        y_gm = asc2.tensor(y, [size])
        for i in asc2.range(size, unroll_factor=2, parallel=True):
            x_val = asc2.load(x_gm, [1], offsets=[i])
            y_val = asc2.load(y_gm, [1], offsets=[i])
            asc2.store(x_val + y_val, y_gm, offsets=[i])

    accumulate[1](torch.zeros(64), torch.zeros(64), 64)
    plan = accumulate.last_plan
    assert plan.pattern == "elementwise:program" and plan.reads == {0, 1} and plan.writes == {1}
    assert len(plan.steps) == 1 and plan.pipeline is None            # the 64 one-element windows merge into one call

    @asc2.jit
    def shifted(x, y, size: int):
        x_gm = asc2.tensor(x, [size])
        y_gm = asc2.tensor(y, [size])
        for i in asc2.range(size - 1):
            asc2.store(asc2.load(x_gm, [1], offsets=[i]) + asc2.load(y_gm, [1], offsets=[i + 1]), y_gm, offsets=[i])

    with pytest.raises(NotImplementedError, match="other positions"):
        shifted[1](torch.zeros(64), torch.zeros(64), 64)
