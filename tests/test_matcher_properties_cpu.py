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


def covered_windows(plan, rows, cols, pitches_of):
    """Rows x cols windows of the general program calls: which output elements they write, and that every operand
    window stays inside its tensor."""
    mask = np.zeros(rows * cols, dtype=bool)
    for step in plan.steps:
        m = re.search(r"over \[(\d+), (\d+)\] pitches \[([\d, ]+)\] from \[([\d, ]*)\] to (\d+)$", step.note)
        assert m, step.note
        r, c = int(m.group(1)), int(m.group(2))
        lds = [int(v) for v in m.group(3).split(",")]
        starts = [int(v) for v in m.group(4).split(",")] + [int(m.group(5))]
        for k, (ld, st0, limit) in enumerate(zip(lds, starts, pitches_of)):
            last = st0 + (r - 1) * ld + c
            assert 0 <= st0 and last <= limit, (step.note, k)        # no operand reads or writes past its tensor
        out_ld, out0 = lds[-1], starts[-1]
        for i in range(r):
            seg = mask[out0 + i * out_ld: out0 + i * out_ld + c]
            assert not seg.any(), step.note                          # no element planned twice
            seg[:] = True
    return mask


@settings(max_examples=60, deadline=None)
@given(rows=st.integers(1, 200), cols=st.sampled_from([8, 64, 136]), rpt=st.sampled_from([1, 3, 8, 32]),
       cores=st.integers(1, 6))
def test_bias_row_plan_with_ragged_tiles_covers_exactly_the_matrix(rows, cols, rpt, cores):
    """x + bias row, rpt rows per tile, blocks striding over the tiles: the last tile usually reaches past the
    matrix; the calls must cover every element once and stay inside x, the bias vector and the result."""
    x = torch.zeros(rows, cols)
    K.add_vector_bias[cores](x, torch.zeros(cols), torch.zeros_like(x), rows, cols, rpt)
    plan = K.add_vector_bias.last_plan
    mask = covered_windows(plan, rows, cols, [rows * cols, cols, rows * cols])
    assert mask.all() and plan.reads == {0, 1} and plan.writes == {2}


@settings(max_examples=40, deadline=None)
@given(n=st.integers(1, 3000), tile=st.sampled_from([8, 64, 256]), shift=st.integers(0, 40), cores=st.integers(1, 5))
def test_shifted_operand_plan_with_a_ragged_tail(n, tile, shift, cores):
    import asc2

    @asc2.jit
    def shifted(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress, n: int, shift: asc.ConstExpr[int],
                tile: asc.ConstExpr[int]):
        x_gm, y_gm, o_gm = asc2.tensor(x_ptr, [n + shift]), asc2.tensor(y_ptr, [n]), asc2.tensor(o_ptr, [n])
        for i in range(asc2.block_idx() * tile, n, asc2.block_num() * tile):
            asc2.store(asc2.load(x_gm, [tile], offsets=[i + shift]) * asc2.load(y_gm, [tile], offsets=[i]), o_gm, offsets=[i])
    shifted[cores](torch.zeros(n + shift), torch.zeros(n), torch.zeros(n), n, shift, tile)
    plan = shifted.last_plan
    mask = np.zeros(n, dtype=bool)
    for step in plan.steps:
        flat = re.search(r"over \[(\d+), (\d+)\)$", step.note)       # operands addressed like the result (shift 0)
        if flat:
            lo, hi = int(flat.group(1)), int(flat.group(2))
            assert shift == 0 and 0 <= lo < hi <= n and not mask[lo:hi].any()
            mask[lo:hi] = True
            continue
        m = re.search(r"over \[(\d+), (\d+)\] pitches \[(\d+), (\d+), (\d+)\] from \[(\d+), (\d+)\] to (\d+)$", step.note)
        assert m, step.note
        r, c, ldx, ldy, ldo, x0, y0, o0 = (int(v) for v in m.groups())
        assert x0 == o0 + shift and y0 == o0 and (r == 1 or ldx == ldy == ldo == c)
        assert x0 + (r - 1) * ldx + c <= n + shift and o0 + (r - 1) * ldo + c <= n
        assert not mask[o0:o0 + r * c].any()
        mask[o0:o0 + r * c] = True
    assert mask.all()
