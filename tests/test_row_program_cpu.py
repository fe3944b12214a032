"""Kernels that reduce their own intermediate tiles along the row (layer norm, normalisations, norms of computed
tiles) on CPU: the launcher compiles them into one row program; evaluated by the CPU oracle it must reproduce
the torch expression.  ``DRY_RUN=1`` stops before the device launch."""
import pytest
import torch

import asc
import asc2

import asc2_scripts as K
from oracle import eltwise as E


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


def decode(step):
    assert step.fn_name == "asc_cuda_row_program"
    ptrs = {i: (i + 1) << 40 for i in range(16)}
    ops, args, n_ops, ins, types, n_in, out, out_type, rows, cols, lds, row_result, _ = step.build(ptrs, None)
    assert len(ops) == n_ops.value
    operands = [((int(a) >> 40) - 1, int(a) & ((1 << 40) - 1)) for a in list(ins)[:n_in.value]]
    return (list(ops), list(args), operands, list(types), ((out.value >> 40) - 1, out.value & ((1 << 40) - 1)),
            out_type.value, rows.value, cols.value, list(lds), row_result.value)


def evaluate(step, runtime_args):
    """The step's effect on its output argument, computed by the oracle from flat views of the arguments."""
    ops, args, operands, types, (out_idx, out_off), out_type, rows, cols, lds, row_result = decode(step)
    inputs = []
    for (idx, byte_off), ld, type_word in zip(operands, lds, types):
        flat = runtime_args[idx].reshape(-1)
        first = byte_off // flat.element_size()
        if type_word & 0x200:       # one element per row
            inputs.append(torch.as_strided(flat, (rows, 1), (ld, 1), first).expand(rows, cols))
        elif ld == 0:
            inputs.append(flat[first:first + cols].expand(rows, cols))
        else:
            inputs.append(torch.as_strided(flat, (rows, cols), (ld, 1), first))
    res = E.run_program(ops, args, inputs, out_type)
    return res[:, 0] if row_result else res


def test_layer_norm_is_one_row_program():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(64, 512, generator=gen) * 2 + 1
    gamma, beta = torch.rand(1, 512, generator=gen) + 0.5, torch.randn(1, 512, generator=gen)
    K.layer_norm_rows[4](x, gamma, beta, torch.empty_like(x), 64, 512, 8, 1e-5)
    plan = K.layer_norm_rows.last_plan
    assert plan.pattern == "row:program" and len(plan.steps) == 1 and not plan.partial_writes
    assert plan.reads == {0, 1, 2} and plan.writes == {3}
    *_, rows, cols, lds, row_result = decode(plan.steps[0])
    assert (rows, cols, lds, row_result) == (64, 512, [512, 0, 0, 512], 0)
    # whole rows of whole tensors: the launcher may stream chunks of rows; gamma and beta stay resident
    pipe = plan.pipeline
    assert pipe is not None and pipe.units == 64 and pipe.resident == {1, 2} and pipe.streamed == {0: 2048, 3: 2048}
    chunk = pipe.make_steps(16, 48)
    assert len(chunk) == 1 and decode(chunk[0])[2][0] == (0, 16 * 2048) and decode(chunk[0])[6] == 32
    ops = decode(plan.steps[0])[0]
    # the centred row is used three times and computed once: two row reductions, one temporary
    assert sum(1 for o in ops if o in (59, 60, 61, 62)) == 2 and ops.count(63) == 1 and ops.count(64) == 2
    out = evaluate(plan.steps[0], [x, gamma, beta, None])
    ref = torch.nn.functional.layer_norm(x, (512, ), gamma[0], beta[0], 1e-5)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)


def test_scalar_reduction_of_a_one_row_tile():
    x = torch.randn(48, 256, generator=torch.Generator().manual_seed(4))
    K.l1_normalize_rows[8](x, torch.empty_like(x), 48, 256)
    plan = K.l1_normalize_rows.last_plan
    assert plan.pattern == "row:program" and len(plan.steps) == 1
    out = evaluate(plan.steps[0], [x, None])
    torch.testing.assert_close(out, x / (x.abs().sum(1, keepdim=True) + 1e-6), rtol=1e-5, atol=1e-6)


def test_per_row_results_of_computed_tiles():
    x = torch.randn(64, 384, generator=torch.Generator().manual_seed(5))
    K.row_sum_of_squares[4](x, torch.empty(64), 64, 384, 8)
    plan = K.row_sum_of_squares.last_plan
    assert plan.pattern == "row:program" and len(plan.steps) == 1 and not plan.partial_writes
    *_, rows, cols, lds, row_result = decode(plan.steps[0])
    assert (rows, cols, lds, row_result) == (64, 384, [384, 1], 1)
    out = evaluate(plan.steps[0], [x, None])
    torch.testing.assert_close(out, x.pow(2).sum(1).sqrt() * 0.5 + x.abs().amax(1), rtol=1e-5, atol=1e-6)


def test_scalar_store_of_reductions_of_a_computed_row():
    x = torch.randn(64, 512, generator=torch.Generator().manual_seed(6))
    K.row_norms_scalar[8](x, torch.empty(64), 64, 512)
    plan = K.row_norms_scalar.last_plan
    assert plan.pattern == "row:program" and len(plan.steps) == 1 and not plan.partial_writes
    *_, rows, cols, lds, row_result = decode(plan.steps[0])
    assert (rows, cols, lds, row_result) == (64, 512, [512, 1], 1)
    out = evaluate(plan.steps[0], [x, None])
    torch.testing.assert_close(out, x.pow(2).sum(1) / 512 + x.abs().amax(1), rtol=1e-5, atol=1e-6)


def test_loaded_columns_repeat_along_the_row():
    gen = torch.Generator().manual_seed(8)
    x, scale, bias = torch.randn(64, 256, generator=gen), torch.randn(64, generator=gen), torch.randn(64, generator=gen)
    K.scale_rows[4](x, scale, bias, torch.empty_like(x), 64, 256, 8)
    plan = K.scale_rows.last_plan
    assert plan.pattern == "row:program" and len(plan.steps) == 1 and not plan.partial_writes
    ops, args, operands, types, _, _, rows, cols, lds, row_result = decode(plan.steps[0])
    assert (rows, cols, lds, row_result) == (64, 256, [256, 1, 1, 256], 0) and types[:3] == [0, 0x200, 0x200]
    out = evaluate(plan.steps[0], [x, scale, bias, None])
    assert torch.equal(out, x * scale[:, None] + bias[:, None])


def test_rows_too_long_for_one_sm_are_refused():
    x = torch.zeros(2, 16384)
    with pytest.raises(NotImplementedError, match="must fit one SM"):
        K.l1_normalize_rows[2](x, torch.empty_like(x), 2, 16384)


def test_golden_fixture_normalisations(golden_dir):
    """The committed float64-derived vectors pin the oracle's rms_norm and the compiled layer-norm program."""
    import os
    import numpy as np
    from oracle import golden
    d = np.load(os.path.join(golden_dir, "normalisation.npz"))
    x, gamma, beta = (torch.from_numpy(d[k]) for k in ("x", "gamma", "beta"))
    eps = float(d["eps"])
    torch.testing.assert_close(golden.rms_norm(x, gamma, eps), torch.from_numpy(d["rms_norm"]), rtol=1e-5, atol=1e-6)
    K.layer_norm_rows[2](x, gamma.reshape(1, -1), beta.reshape(1, -1), torch.empty_like(x), 8, 512, 4, eps)
    out = evaluate(K.layer_norm_rows.last_plan.steps[0], [x, gamma.reshape(1, -1), beta.reshape(1, -1), None])
    torch.testing.assert_close(out, torch.from_numpy(d["layer_norm"]), rtol=1e-5, atol=2e-6)
