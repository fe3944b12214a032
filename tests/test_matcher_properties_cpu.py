"""Property tests of the launch planner: for random sizes, tile shapes and block counts the element set the
planned C-ABI calls cover must equal the set a block-by-block execution of the kernel would store
(loads pad, stores clip: lib/Conversion/LowerToAsc/LowerAscTileDataTransfer.cpp:184-218,254-261).
``DRY_RUN=1`` stops before the device launch."""
import re

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

import asc

import asc2_scripts as K


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


def covered_flat(plan, numel):
    mask = np.zeros(numel, dtype=bool)
    for step in plan.steps:
        m = re.search(r"\[(\d+), (\d+)\)$", step.note)
        assert m, step.note
        lo, hi = int(m.group(1)), int(m.group(2))
        assert 0 <= lo < hi <= numel and not mask[lo:hi].any()       # in bounds, no element planned twice
        mask[lo:hi] = True
    return mask


@settings(max_examples=60, deadline=None)
@given(size=st.integers(1, 5000), tile=st.sampled_from([8, 16, 64, 128, 1000]), cores=st.integers(1, 9),
       per_block=st.integers(1, 7))
def test_vadd_plan_covers_exactly_what_the_blocks_store(size, tile, cores, per_block):
    x = np.zeros(size, np.float32)
    K.vadd[cores](x, x, x.copy(), size, tile, per_block)
    want = np.zeros(size, dtype=bool)
    for block in range(cores):
        for i in range(per_block):
            off = block * tile * per_block + i * tile
            want[off:off + tile] = True                              # slicing clips like the store does
    if not want.any():
        return
    plan = K.vadd.last_plan
    assert np.array_equal(covered_flat(plan, size), want)
    assert (plan.partial_writes == set()) == bool(want.all())


@settings(max_examples=40, deadline=None)
@given(rows=st.integers(1, 300), cols=st.sampled_from([8, 64, 256]), cores=st.integers(1, 7))
def test_softmax_rows_plan_covers_every_row_once(rows, cols, cores):
    x = torch.zeros(rows, cols)
    K.softmax_rows[cores](x, torch.empty_like(x), rows, cols, tile_size=cols)
    notes = [s.note for s in K.softmax_rows.last_plan.steps]
    assert notes == [f"rows [0, {rows}) x {cols} cols"]              # block-strided rows merge into one call


@settings(max_examples=40, deadline=None)
@given(rows=st.integers(1, 200), cols=st.integers(1, 40).map(lambda c: 8 * c), tile_r=st.sampled_from([1, 4, 16, 33]),
       tile_c=st.sampled_from([8, 32, 64]), cores=st.integers(1, 6))
def test_2d_tile_grid_plan_covers_the_matrix(rows, cols, tile_r, tile_c, cores):
    x = torch.zeros(rows, cols)
    K.scale_2d_tiles[cores](x, torch.zeros_like(x), rows, cols, 0.5, tile_r, tile_c)
    plan = K.scale_2d_tiles.last_plan
    mask = np.zeros((rows, cols), dtype=bool)
    for step in plan.steps:
        flat = re.search(r"over \[(\d+), (\d+)\)$", step.note)
        win = re.search(r"over \[(\d+), (\d+)\] at \((\d+), (\d+)\)$", step.note)
        if flat:
            lo, hi = int(flat.group(1)), int(flat.group(2))
            assert not mask.reshape(-1)[lo:hi].any()
            mask.reshape(-1)[lo:hi] = True
        else:
            r, c, r0, c0 = (int(g) for g in win.groups())
            assert r0 + r <= rows and c0 + c <= cols and not mask[r0:r0 + r, c0:c0 + c].any()
            mask[r0:r0 + r, c0:c0 + c] = True
    assert mask.all()                                                # the blocks walk the whole tile grid


@settings(max_examples=30, deadline=None)
@given(m_tiles=st.integers(1, 4), n_tiles=st.integers(1, 4), k=st.sampled_from([64, 128]), cores=st.sampled_from([1, 2, 4]))
def test_matmul_blocked_plan_is_one_gemm(m_tiles, n_tiles, k, cores):
    m_tile, n_tile = 32, 64
    m, n = m_tiles * m_tile, n_tiles * n_tile
    if (m_tiles * n_tiles) % cores:
        return
    per_core = m_tiles * n_tiles // cores
    ntpb = next(d for d in range(min(n_tiles, per_core), 0, -1) if n_tiles % d == 0 and per_core % d == 0)
    if m_tiles % (per_core // ntpb):
        return
    a, b = torch.zeros(m, k, dtype=torch.float16), torch.zeros(k, n, dtype=torch.float16)
    mtpb = K.mn_tiles_per_block(m, n, cores, m_tile, n_tile, ntpb)
    K.matmul_mn_blocked[cores](a, b, torch.zeros(m, n), a.shape, b.shape, (m, n), m_tile, mtpb, n_tile, ntpb)
    plan = K.matmul_mn_blocked.last_plan
    assert len(plan.steps) == 1 and plan.steps[0].fn_name == "asc_cuda_gemm_f16" and not plan.partial_writes
