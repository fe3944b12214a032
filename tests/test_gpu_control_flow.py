"""Control flow on the GPU: ``if`` on the block index or a loop variable, and tiles carried from one loop iteration
to the next, against torch on the same inputs (the kernels are those of tests/test_branches_cpu.py and the
running sum of tests/test_eltwise_cpu.py)."""
import pytest
import torch

import asc
import asc.runtime.config as config
import asc2

import test_branches_cpu as B

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id, monkeypatch):
    monkeypatch.delenv("DRY_RUN", raising=False)
    config.set_platform(backend, platform, device_id)


@pytest.mark.parametrize("cores", [1, 3, 8])
def test_even_and_odd_tiles_take_different_arms(cores):
    n, tiles = 64, 8
    x = torch.randn(tiles * n, generator=torch.Generator().manual_seed(cores))
    out = torch.full_like(x, -9.0)
    B.even_odd[cores](x, out, n, tiles)
    want = x.view(tiles, n).clone()
    want[0::2] *= 2
    want[1::2] += 1
    assert torch.equal(out, want.view(-1))


def test_nested_branches_on_the_block_index():
    n = 64
    x = torch.randn(8 * n, generator=torch.Generator().manual_seed(5))
    out = torch.full_like(x, -9.0)
    B.first_blocks_only[4](x, out, n, 3)
    xv, want = x.view(8, n), torch.full((8, n), -9.0)
    want[0] = xv[0] - 1
    want[1:3] = torch.exp(xv[1:3])
    want[4:8] = xv[0:4]
    torch.testing.assert_close(out.view(8, n), want, rtol=2e-6, atol=0)
    assert torch.equal(out.view(8, n)[3], want[3])            # block 3 is not among the active ones: untouched


@asc2.jit
def running_sum(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int], reps: int):
    x_gm = asc2.tensor(x_ptr, [reps * n])
    acc = asc2.zeros([n], dtype=asc.float32)
    for i in range(reps):
        acc = acc + asc2.load(x_gm, [n], offsets=[i * n])
    asc2.store(acc, asc2.tensor(out_ptr, [n]), offsets=[0])


@pytest.mark.parametrize("reps", [1, 4, 5])
def test_tile_carried_across_iterations(reps):
    n = 4096
    x = torch.randn(reps * n, generator=torch.Generator().manual_seed(reps))
    out = torch.zeros(n)
    running_sum[1](x, out, n, reps)
    want = torch.zeros(n)
    for i in range(reps):                       # the kernel's own order of additions
        want = want + x[i * n:(i + 1) * n]
    assert torch.equal(out, want)


@asc2.jit
def masked_ops(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: asc.ConstExpr[int], cols: asc.ConstExpr[int],
               tiles: int, count: int):
    x_gm, out_gm = asc2.tensor(x_ptr, [tiles * rows, cols]), asc2.tensor(out_ptr, [tiles * rows, cols])
    for t in range(asc2.block_idx(), tiles, asc2.block_num()):
        x = asc2.load(x_gm, [rows, cols], offsets=[t * rows, 0])
        with asc2.mask(count=count, other=0.5):
            y = asc2.exp(x) + 1              # both operations keep `count` elements of the tile and fill the rest
        asc2.store(y * 2, out_gm, offsets=[t * rows, 0])


@pytest.mark.parametrize("rows, cols, count", [(1, 256, 100), (4, 64, 130), (8, 1024, 8192), (2, 512, 0)])
def test_count_mask_keeps_the_first_elements_of_every_tile(rows, cols, count):
    tiles = 6
    x = torch.randn(tiles * rows, cols, generator=torch.Generator().manual_seed(count))
    out = torch.zeros_like(x)
    masked_ops[4](x, out, rows, cols, tiles, count)
    active = (torch.arange(rows * cols) < count).reshape(rows, cols).repeat(tiles, 1)
    inner = torch.where(active, torch.exp(x), torch.tensor(0.5))          # exp under the mask
    want = torch.where(active, inner + 1, torch.tensor(0.5)) * 2          # + 1 under the mask, * 2 outside it
    torch.testing.assert_close(out, want, rtol=2e-6, atol=0)


def _leaky(t, slope):
    """A Python helper called from kernels: it is traced like the kernel's own statements."""
    return asc2.where(t >= 0, t, t * slope)


@asc2.jit
def spare_blocks_return_early(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, flag_ptr: asc.GlobalAddress, n: int,
                              tile: asc.ConstExpr[int], active: int):
    if asc2.block_idx() >= active:
        return
    x_gm, out_gm, flag_gm = asc2.tensor(x_ptr, [n]), asc2.tensor(out_ptr, [n]), asc2.tensor(flag_ptr, [tile])
    if asc2.block_idx() == 0:
        asc2.store(asc2.full([tile], 1.0, dtype=asc.float32), flag_gm, offsets=[0])
    for i in range(asc2.block_idx() * tile, n, active * tile):
        if i + tile <= n:                                         # the ragged tail is left alone
            asc2.store(_leaky(asc2.load(x_gm, [tile], offsets=[i]), 0.2), out_gm, offsets=[i])


def test_early_return_helper_function_and_a_guarded_tail():
    n, tile = 5000, 256
    x = torch.randn(n, generator=torch.Generator().manual_seed(14))
    out, flag = torch.full((n, ), 7.0), torch.zeros(tile)
    spare_blocks_return_early[8](x, out, flag, n, tile, 3)
    plan = spare_blocks_return_early.last_plan
    full = (n // tile) * tile
    want = torch.full((n, ), 7.0)
    want[:full] = torch.where(x[:full] >= 0, x[:full], x[:full] * 0.2)
    assert torch.equal(out, want) and bool((flag == 1).all())
    # the loop's store is traced on both sides of `if block_idx() == 0` and merges back into one effect: two kernels
    assert len(plan.steps) == 2, [s.note for s in plan.steps]
