"""Kernels specialised at first use, on CPU: the words a program is keyed by, the generated translation unit, the
nvcc build into the file cache (nvcc cross-compiles without a GPU), loading and registering the library, and the
plan steps that ask for it.  ``DRY_RUN=1`` stops before any device launch."""
import os

import pytest
import torch

import asc
import asc2
from pyasc_b200 import jit


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


def test_program_words_carry_operand_indices_and_row_flags():
    # LOAD 1, LOAD 0 (one element per row), SUB, TEE 2, ROW_SUM, TMP 2, MUL | IMM
    ops, args = [0, 0, 3, 63, 59, 64, 4 | 0x100], [1, 0, 0, 2, 0, 2, 1065353216]
    assert jit.program_words(ops, args, [True, False]) == (1 << 16, 0 | (1 << 24), 3, 63 | (2 << 16), 59, 64 | (2 << 16),
                                                           4 | 0x100)
    assert jit.program_words(ops, args) == (1 << 16, 0, 3, 63 | (2 << 16), 59, 64 | (2 << 16), 4 | 0x100)
    assert [jit.row_kind(c) for c in (1, 256, 257, 1024, 4096, 8192)] == [1001, 1001, 1002, 1004, 1016, 1032]


def test_generated_unit_instantiates_the_right_executor():
    src = jit.source(0, (0, 11, 258))
    assert "OpList<0, 11, 258>" in src and "jit_launch_eltwise<P>" in src and 'extern "C" int asc_jit_run' in src
    assert "jit_launch_row<P, 16>" in jit.source(jit.ROW_KIND + 16, (0, 59))
    # the cache key covers the program, its kind and the device code it is built from
    assert jit.library_name(0, (0, 11)) != jit.library_name(0, (0, 12)) != jit.library_name(1001, (0, 12))


@asc2.jit
def softsign_rows(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, cols: asc.ConstExpr[int]):
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(out_ptr, [rows, cols])
    for i in range(asc2.block_idx(), rows, asc2.block_num()):
        x = asc2.load(x_gm, [1, cols], offsets=[i, 0])
        asc2.store(x / (asc2.abs(x) + 1), out_gm, offsets=[i, 0])


@asc2.jit
def centre_rows(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, cols: asc.ConstExpr[int]):
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(out_ptr, [rows, cols])
    for i in range(asc2.block_idx(), rows, asc2.block_num()):
        x = asc2.load(x_gm, [1, cols], offsets=[i, 0])
        asc2.store(x - asc2.reduce_sum(x) / cols, out_gm, offsets=[i, 0])


def test_plan_steps_name_their_program():
    x = torch.zeros(8, 1024)
    softsign_rows[4](x, torch.zeros_like(x), 8, 1024)
    (step, ) = softsign_rows.last_plan.steps
    assert step.program[0] == 0 and step.program[1] == jit.program_words(*_ops_args(step))
    centre_rows[4](x, torch.zeros_like(x), 8, 1024)
    (step, ) = centre_rows.last_plan.steps
    assert step.program[0] == jit.ROW_KIND + 4 and 59 in step.program[1]


def _ops_args(step):
    built = step.build({0: 0, 1: 0}, None)
    n = built[2].value
    return list(built[0][:n]), list(built[1][:n])


def test_build_load_register_and_cache(tmp_path, monkeypatch):
    if jit.compiler() is None:
        pytest.skip("no nvcc on this machine")
    monkeypatch.setenv("PYASC_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("ASC_CUDA_JIT", "sync")
    x = torch.zeros(8, 1024)
    centre_rows[4](x, torch.zeros_like(x), 8, 1024)
    kind, words = centre_rows.last_plan.steps[0].program
    words = words + ()                               # a key of its own for this test: same program, fresh cache
    assert not list(tmp_path.iterdir())
    assert jit.request(kind, words, wait=True), jit.failures()
    (lib, ) = list(tmp_path.iterdir())               # one library, no temporary files left behind
    assert lib.name == jit.library_name(kind, words) and str(lib) in jit.builds
    stamp = lib.stat().st_mtime_ns
    assert jit.request(kind, words)                  # registered: nothing to do
    assert jit.build_library(kind, words) == lib and lib.stat().st_mtime_ns == stamp     # a cache hit does not rebuild
    monkeypatch.setenv("ASC_CUDA_JIT", "0")
    assert not jit.request(0, (0, 9))                # switched off: the interpreter keeps the program
