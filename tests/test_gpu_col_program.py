"""Reductions of computed tiles along the first axis, and of fp16 / bf16 tiles along either axis, on the GPU.

``asc2.reduce_*(expression, 0)`` (python/asc/language/tile/reduction_ops.py:33-188 in the reference; shapes and
distributions after python/test/asc2/operations/test_reduce_ops.py:17-104) runs as one column program per tile
(``asc_cuda_col_program``); 16-bit tiles reduced along the rows run as row programs.  The device result is compared
with the CPU evaluation of the same program (oracle.eltwise) reduced by torch: max / min bit-exact, sums and products
within the rounding of a different summation order, 16-bit results after one rounding of the fp32 combination."""
import ctypes
import struct

import pytest
import torch

import asc
import asc.runtime.config as config
import asc2

from oracle import eltwise as E
from pyasc_b200 import capi

pytestmark = pytest.mark.gpu

TYPE_OF = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int32: 3}
REDUCERS = {0: lambda t: t.sum(0), 1: lambda t: t.amax(0), 2: lambda t: t.amin(0), 3: lambda t: t.prod(0)}


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id):
    config.set_platform(backend, platform, device_id)


@pytest.fixture(scope="module")
def lib():
    torch.cuda.set_device(0)
    return capi.load()


def fbits(v: float) -> int:
    return struct.unpack("<i", struct.pack("<f", v))[0]


def col_program(lib, ops, args, inputs, lds, out, rows, cols, kind, expect=0):
    ops_a, args_a = (ctypes.c_int32 * len(ops))(*ops), (ctypes.c_int32 * len(args))(*args)
    ins = (ctypes.c_void_p * max(1, len(inputs)))(*[t.data_ptr() for t in inputs])
    types = (ctypes.c_int32 * max(1, len(inputs)))(*[TYPE_OF[t.dtype] for t in inputs])
    lds_a = (ctypes.c_int64 * max(1, len(lds)))(*lds)
    rc = lib.asc_cuda_col_program(ops_a, args_a, len(ops), ins, types, len(inputs), ctypes.c_void_p(out.data_ptr()),
                                  TYPE_OF[out.dtype], rows, cols, lds_a, kind, None)
    assert rc == expect, f"returned {rc}: {capi.status_string(rc)} {capi.last_cuda_error()}"
    if rc == 0:
        capi.check_device_status(None)


# (x * w)^2 - 0.25 with w one row broadcast over the window: LOAD x, LOAD w, MUL, TEE-free square by reloading
SQUARE_OPS = [0, 0, 4, 0, 0, 4, 4, 3 | 0x100]
SQUARE_ARGS = [0, 1, 0, 0, 1, 0, 0, fbits(0.25)]          # SUB|IMM: 0.25 - value


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("rows, cols, pad", [(1, 1, 0), (32, 256, 0), (64, 33, 7), (7, 5000, 0), (300, 1024, 16)])
def test_capi_column_programs_equal_the_oracle(lib, dtype, rows, cols, pad):
    gen = torch.Generator().manual_seed(rows * 131 + cols)
    ld = cols + pad
    x = (torch.randn(rows, ld, generator=gen) * 0.8).to(dtype)
    w = (torch.rand(1, cols, generator=gen) + 0.5).to(dtype)
    xd, wd = x.cuda(), w.cuda()
    ops, args = list(SQUARE_OPS), list(SQUARE_ARGS)
    if dtype != torch.float32:          # every intermediate takes the tile's type, as the launcher's programs do
        rnd = 33 if dtype == torch.float16 else 34
        ops = [0, 0, 4, rnd, 0, 0, 4, rnd, 4, rnd, 3 | 0x100, rnd]
        args = [0, 1, 0, 0, 0, 1, 0, 0, 0, 0, fbits(0.25), 0]
    value = E.run_program(ops, args, [x[:, :cols], w.expand(rows, cols)], 0)
    for kind in range(4):
        out = torch.full((cols + 1, ), 7.0, dtype=dtype, device="cuda")
        col_program(lib, ops, args, [xd, wd], [ld, 0], out, rows, cols, kind)
        got = out.cpu()
        assert got[cols] == 7.0                                        # nothing written past the columns
        want = REDUCERS[kind](value.float())
        if kind in (1, 2):
            assert torch.equal(got[:cols], want.to(dtype)), kind
        else:
            tol = 2e-5 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1.6e-2)
            torch.testing.assert_close(got[:cols].float(), want.to(dtype).float(), rtol=tol, atol=tol)


def test_capi_column_program_nan_identity_and_rejections(lib):
    x = torch.randn(40, 300)
    x[5, ::9] = float("nan")
    xd = x.cuda()
    out = torch.zeros(300, device="cuda")
    for kind in (1, 2):                                   # max / min carry a NaN of the column, like torch.amax
        col_program(lib, [0], [0], [xd], [300], out, 40, 300, kind)
        want = REDUCERS[kind](x)
        got = out.cpu()
        assert torch.equal(got.isnan(), want.isnan()) and bool(want.isnan().any())
        assert torch.equal(got[~want.isnan()], want[~want.isnan()])
    # no rows: every column receives the identity of the reduction
    for kind, identity in ((0, 0.0), (1, float("-inf")), (2, float("inf")), (3, 1.0)):
        col_program(lib, [0], [0], [xd], [300], out, 0, 300, kind)
        assert bool((out.cpu() == identity).all())
    col_program(lib, [0], [0], [xd], [300], out, 40, 0, 0)                   # no columns: nothing to do
    col_program(lib, [0], [0], [xd], [300], out, 40, 300, 4, expect=1)       # unknown reduction
    col_program(lib, [0], [0], [xd], [299], out, 40, 300, 0, expect=1)       # pitch shorter than a row
    col_program(lib, [0, 2], [0, 0], [xd], [300], out, 40, 300, 0, expect=1)  # malformed program
    iout = torch.zeros(300, dtype=torch.int32, device="cuda")
    col_program(lib, [0], [0], [xd], [300], iout, 40, 300, 0, expect=3)      # integer combination: unsupported


@asc2.jit
def col_norms(x_ptr: asc.GlobalAddress, w_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, tiles: int,
              rows: asc.ConstExpr[int], cols: asc.ConstExpr[int], op: asc.ConstExpr):
    x_gm = asc2.tensor(x_ptr, [tiles * rows, cols])
    out_gm = asc2.tensor(out_ptr, [tiles, cols])
    w = asc2.load(asc2.tensor(w_ptr, [1, cols]), [1, cols], offsets=[0, 0])
    for t in range(asc2.block_idx(), tiles, asc2.block_num()):
        x = asc2.load(x_gm, [rows, cols], offsets=[t * rows, 0])
        y = x * w.broadcast_to(rows, cols)
        asc2.store(op(y * y + 0.5, 0, keep_dims=True), out_gm, offsets=[t, 0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("op, torch_op", [(asc2.reduce_sum, torch.sum), (asc2.reduce_max, torch.amax),
                                          (asc2.reduce_min, torch.amin)], ids=lambda v: getattr(v, "__name__", ""))
def test_column_reduction_of_an_expression_through_asc2(op, torch_op, dtype):
    tiles, rows, cols = 6, 32, 256
    gen = torch.Generator().manual_seed(11)
    x = (torch.randn(tiles * rows, cols, generator=gen) * 0.5).to(dtype)
    w = (torch.rand(1, cols, generator=gen) + 0.5).to(dtype)
    out = torch.zeros(tiles, cols, dtype=dtype)
    col_norms[4](x, w, out, tiles, rows, cols, op)
    assert col_norms.last_plan.pattern.endswith(":columns")
    y = x * w                                            # torch rounds every intermediate to the tile's type too
    value = (y * y + 0.5).reshape(tiles, rows, cols)
    if op is asc2.reduce_sum:
        want = value.float().sum(1).to(dtype)
        tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
        torch.testing.assert_close(out.float(), want.float(), rtol=tol, atol=tol)
    else:
        assert torch.equal(out, torch_op(value, 1))


@asc2.jit
def row_reduce(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, cols: asc.ConstExpr[int],
               rpt: asc.ConstExpr[int], op: asc.ConstExpr):
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(out_ptr, [rows])
    for i in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
        asc2.store(op(asc2.load(x_gm, [rpt, cols], offsets=[i, 0]), 1), out_gm, offsets=[i])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("op, torch_op", [(asc2.reduce_sum, torch.sum), (asc2.reduce_max, torch.amax),
                                          (asc2.reduce_min, torch.amin), (asc2.reduce_prod, torch.prod)],
                         ids=lambda v: getattr(v, "__name__", ""))
def test_half_precision_row_reductions_through_asc2(op, torch_op, dtype):
    rows, cols = 128, 512
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(rows, cols, generator=gen)
    if op is asc2.reduce_prod:
        x = 1.0 + x * 0.01                              # keeps the product of 512 factors in range
    x = x.to(dtype)
    out = torch.zeros(rows, dtype=dtype)
    row_reduce[8](x, out, rows, cols, 16, op)
    assert row_reduce.last_plan.steps[0].fn_name == "asc_cuda_row_program"
    want = torch_op(x.float(), 1).to(dtype)             # fp32 combination, one rounding to the tile's type
    if op in (asc2.reduce_max, asc2.reduce_min):
        assert torch.equal(out, want)
    else:
        tol = 2e-3 if dtype == torch.float16 else 1.6e-2
        torch.testing.assert_close(out.float(), want.float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("op, torch_op", [(asc2.reduce_sum, torch.sum), (asc2.reduce_max, torch.amax),
                                          (asc2.reduce_min, torch.amin), (asc2.reduce_prod, torch.prod)],
                         ids=lambda v: getattr(v, "__name__", ""))
def test_whole_tile_reductions_of_half_precision_tiles(op, torch_op, dtype, lib):
    """asc2.reduce_*(tile) without dimensions on a 16-bit tile, stored through asc2.full (the reference's
    test_reduce_all body, python/test/asc2/operations/test_reduce_ops.py, with a 16-bit dtype)."""
    import asc2_scripts as K
    gen = torch.Generator().manual_seed(21)
    x = torch.randn(32, 32, generator=gen)
    if op is asc2.reduce_prod:
        x = 1.0 + x * 0.02
    x = x.to(dtype)
    out = torch.zeros(32, dtype=dtype)
    K.reduce_all[1](x, out, [32, 32], [0, 0], [32], [0], op)
    want = torch_op(x.float()).to(dtype)
    if op in (asc2.reduce_max, asc2.reduce_min):
        assert torch.equal(out, want.expand(32))
    else:
        tol = 2e-3 if dtype == torch.float16 else 1.6e-2
        torch.testing.assert_close(out.float(), want.float().expand(32), rtol=tol, atol=tol)
    # the C ABI directly: a window inside a wider matrix, NaN propagation of max, rejections
    xd = torch.randn(40, 72, generator=gen).to(dtype).cuda()
    od = torch.full((9, ), 7.0, dtype=dtype, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    dt = 1 if dtype == torch.bfloat16 else 0
    assert lib.asc_cuda_reduce_all_f16(P(xd), P(od), 40, 64, 72, 0, 8, dt, None) == 0
    capi.check_device_status(None)
    want = xd[:, :64].float().sum().to(dtype)
    tol = 4e-3 if dtype == torch.float16 else 3e-2
    torch.testing.assert_close(od[:8].float().cpu(), want.float().cpu().expand(8), rtol=tol, atol=tol)
    assert od[8].item() == 7.0
    xd[3, 5] = float("nan")
    assert lib.asc_cuda_reduce_all_f16(P(xd), P(od), 40, 64, 72, 1, 1, dt, None) == 0
    assert bool(od[0].isnan())
    assert lib.asc_cuda_reduce_all_f16(P(xd), P(od), 40, 64, 72, 0, 0, dt, None) == 0        # nothing to fill
    assert lib.asc_cuda_reduce_all_f16(P(xd), P(od), 40, 64, 63, 0, 1, dt, None) == 1        # pitch shorter than a row
    assert lib.asc_cuda_reduce_all_f16(P(xd), P(od), 40, 64, 72, 0, 1, 2, None) == 1         # unknown element type
    assert lib.asc_cuda_reduce_all_f16(P(xd), P(od), 1 << 13, 1 << 12, 1 << 12, 0, 1, dt, None) == 6   # larger than a tile


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=str)
def test_softmax_and_standardisation_down_the_columns(dtype):
    """Reductions along the first axis used inside the expression (`x - reduce_max(x, 0, keep_dims=True)
    .broadcast_to(...)`): each is computed into a temporary first, then read back as a broadcast row."""
    import asc2_scripts as K
    tiles, rows, cols = 4, 64, 256
    gen = torch.Generator().manual_seed(12)
    x = torch.randn(tiles * rows, cols, generator=gen).to(dtype)
    out = torch.zeros_like(x)
    K.column_softmax[2](x, out, tiles, rows, cols)
    assert K.column_softmax.last_plan.pattern == "column:statistics"
    want = torch.softmax(x.float().reshape(tiles, rows, cols), dim=1).reshape(tiles * rows, cols)
    tol = 1e-5 if dtype == torch.float32 else 2e-3
    torch.testing.assert_close(out.float(), want, rtol=tol, atol=tol)
    out2 = torch.zeros_like(x)
    K.column_standardise[2](x, out2, tiles, rows, cols, 1e-5)
    t = x.float().reshape(tiles, rows, cols)
    d = t - t.mean(1, keepdim=True)
    want2 = (d * torch.rsqrt((d * d).mean(1, keepdim=True) + 1e-5)).reshape(tiles * rows, cols)
    tol = 1e-5 if dtype == torch.float32 else 4e-3
    torch.testing.assert_close(out2.float(), want2, rtol=tol, atol=tol)
