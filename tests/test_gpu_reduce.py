"""Reductions on the GPU: the reference's operation tests through the asc2 surface
(python/test/asc2/operations/test_reduce_ops.py:17-104, test_softmax.py: same shapes, distributions and
torch goldens) and the C-ABI entry point at sizes beyond L2.  max / min are bit-exact; sums and products
are compared with torch's CPU result within the rounding of a different summation order."""
import ctypes

import pytest
import torch

import asc.runtime.config as config
import asc2

import asc2_scripts as K
from oracle import golden
from pyasc_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id):
    config.set_platform(backend, platform, device_id)


REDUCE_CASES = [
    (asc2.reduce_prod, torch.prod, False, 0), (asc2.reduce_prod, torch.prod, False, 1),
    (asc2.reduce_min, torch.amin, False, 0), (asc2.reduce_min, torch.amin, False, 1),
    (asc2.reduce_sum, torch.sum, False, 0), (asc2.reduce_sum, torch.sum, False, 1),
    (asc2.reduce_max, torch.amax, False, 0), (asc2.reduce_max, torch.amax, False, 1),
    (asc2.reduce_prod, torch.prod, True, 0), (asc2.reduce_sum, torch.sum, True, 0),
]


@pytest.mark.parametrize("op, torch_op, keep_dims, dim", REDUCE_CASES, ids=lambda v: getattr(v, "__name__", str(v)))
def test_reduce(op, torch_op, keep_dims, dim):
    shape = [64, 32]
    gen = torch.Generator().manual_seed(2026)
    x = torch.randn(shape, generator=gen) * 2.0
    output_shape = list(shape)
    if keep_dims:
        output_shape[dim] = 1
    else:
        del output_shape[dim]
    output = torch.zeros(output_shape)
    K.reduce_axis[1](x, output, dim, shape, [0, 0], output_shape, [0] * len(output_shape), op, keep_dims)
    expected = torch_op(x, dim, keepdim=keep_dims)
    if op in (asc2.reduce_max, asc2.reduce_min):
        assert torch.equal(output, expected)
    else:
        # a product of 32 or 64 factors accumulates one rounding per factor in either order
        torch.testing.assert_close(output, expected, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("op, torch_op", [(asc2.reduce_sum, torch.sum), (asc2.reduce_max, torch.amax),
                                          (asc2.reduce_min, torch.amin), (asc2.reduce_prod, torch.prod)],
                         ids=lambda v: getattr(v, "__name__", str(v)))
def test_reduce_all(op, torch_op):
    gen = torch.Generator().manual_seed(7)
    x = torch.randn([32, 32], generator=gen) * (1.05 if op is asc2.reduce_prod else 2.0)
    out = torch.zeros(32)
    K.reduce_all[1](x, out, [32, 32], [0, 0], [32], [0], op)
    expected = torch.ones(32) * torch_op(x).item()
    torch.testing.assert_close(out, expected, rtol=2e-5, atol=1e-5)


@pytest.mark.parametrize("tile_size", [1, 7, 17])
def test_reduce_partial_tile(tile_size):
    torch.manual_seed(0)
    x = torch.rand(32, dtype=torch.float32) * -10.0
    x[tile_size:] = 1000.0
    out = torch.empty(1, dtype=torch.float32)
    K.reduce_tile[1](x, out, 32, tile_size=tile_size)
    torch.testing.assert_close(out, torch.amax(x[:tile_size]).unsqueeze(0), rtol=0, atol=0)


def test_row_sums_over_all_blocks():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(4096, 1024, generator=gen)
    out = torch.full((4096, ), -1.0)
    K.row_sums[16](x, out, 4096, 1024, 8)
    torch.testing.assert_close(out, x.sum(1), rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(out, x.double().sum(1).float(), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("dtype, shape", [(torch.float16, [1, 16]), (torch.float16, [4, 1024]), (torch.float32, [1, 8]),
                                          (torch.float32, [4, 256])])
def test_softmax_2d_op(dtype, shape):
    src = torch.rand(shape, dtype=dtype)
    keep = src.clone()
    dst = torch.zeros_like(src)
    K.softmax_2d[1](dst, src, shape)
    torch.testing.assert_close(dst, torch.softmax(keep, dim=1))
    assert torch.equal(src, keep)                      # the tile stored back to the source is unchanged


@pytest.mark.parametrize("dtype, length", [(torch.float16, 16), (torch.float16, 1024), (torch.float32, 8),
                                           (torch.float32, 1024)])
def test_softmax_1d_op(dtype, length):
    src = torch.rand(length, dtype=dtype)
    dst = torch.zeros_like(src)
    K.softmax_1d[1](dst, src, length)
    torch.testing.assert_close(dst, torch.softmax(src, dim=0))


# ------------------------------------------------------------------------------- C ABI
@pytest.fixture(scope="module")
def lib():
    torch.cuda.set_device(0)
    return capi.load()


def call(lib, x, out, rows, cols, ld, axis, kind, n_fill=1, expect=0):
    rc = lib.asc_cuda_reduce_f32(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, cols, ld, axis,
                                 kind, n_fill, None)
    assert rc == expect, f"returned {rc}: {capi.status_string(rc)} {capi.last_cuda_error()}"
    if rc == 0:
        capi.check_device_status(None)


@pytest.mark.parametrize("rows, cols", [(1, 1), (3, 5), (1000, 33), (257, 4096), (65536, 1024), (37, 100003)])
def test_capi_row_and_column_reductions(lib, rows, cols):
    """Includes a 256 MiB window (beyond L2), rows long enough for the CTA-per-row kernel and ragged sizes."""
    gen = torch.Generator(device="cuda").manual_seed(rows * 31 + cols)
    x = torch.randn(rows, cols + 3, device="cuda", generator=gen)      # pitch != cols
    win = x[:, :cols]
    for axis, n_out in ((1, rows), (0, cols)):
        out = torch.full((n_out + 1, ), 7.0, device="cuda")
        call(lib, x, out, rows, cols, cols + 3, axis, 1)
        assert torch.equal(out[:n_out], win.amax(dim=axis)) and out[n_out] == 7.0
        call(lib, x, out, rows, cols, cols + 3, axis, 2)
        assert torch.equal(out[:n_out], win.amin(dim=axis))
        call(lib, x, out, rows, cols, cols + 3, axis, 0)
        ref = win.double().sum(dim=axis)
        scale = win.abs().double().sum(dim=axis).clamp_min(1e-30)
        assert float(((out[:n_out].double() - ref).abs() / scale).max()) < 2e-6     # error relative to sum |x|
    small = (torch.rand(rows, min(cols, 64), device="cuda", generator=gen) * 0.2 + 0.9).contiguous()
    out = torch.empty(rows, device="cuda")
    call(lib, small, out, rows, small.shape[1], small.shape[1], 1, 3)
    torch.testing.assert_close(out, small.double().prod(dim=1).float(), rtol=1e-5, atol=0)


def test_capi_max_min_reductions_propagate_nan(lib):
    """torch.amax / amin return NaN for a row or column that holds one; so do the kernels (all four of them:
    a warp per row, a CTA per row, along columns, the whole window)."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    for rows, cols in ((37, 100), (5, 20000)):
        x = torch.randn(rows, cols, device="cuda", generator=gen)
        x[2, cols // 3] = float("nan")
        for axis, n_out in ((1, rows), (0, cols)):
            for kind, ref in ((1, x.amax(dim=axis)), (2, x.amin(dim=axis))):
                out = torch.zeros(n_out, device="cuda")
                call(lib, x, out, rows, cols, cols, axis, kind)
                assert torch.equal(out.isnan(), ref.isnan()) and int(ref.isnan().sum()) == 1
                assert torch.equal(out[~ref.isnan()], ref[~ref.isnan()])
    x = torch.randn(64, 64, device="cuda", generator=gen)
    x[10, 10] = float("nan")
    out = torch.zeros(1, device="cuda")
    call(lib, x, out, 64, 64, 64, -1, 1)
    assert bool(out.isnan().all())


def test_capi_full_reduction_and_rejections(lib):
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(512, 1000, device="cuda", generator=gen)
    out = torch.zeros(40, device="cuda")
    call(lib, x, out, 512, 1000, 1000, -1, 1, n_fill=33)
    assert torch.equal(out[:33], x.max().expand(33)) and bool((out[33:] == 0).all())
    call(lib, x, out, 512, 1000, 1000, -1, 0, n_fill=1)
    assert abs(float(out[0]) - float(x.double().sum())) < 1e-2
    call(lib, x, out, 0, 1000, 1000, 1, 0)                              # nothing to write
    call(lib, x, out, 512, 1000, 999, 1, 0, expect=1)                   # pitch smaller than the row
    call(lib, x, out, 512, 1000, 1000, 2, 0, expect=1)                  # no such axis
    call(lib, x, out, 512, 1000, 1000, 1, 4, expect=1)                  # no such kind
    call(lib, x, out, 1 << 13, 1 << 12, 1 << 12, -1, 0, expect=6)       # a full reduction is for tile-sized windows


def test_row_sums_pinned_pipelined_matches_plain():
    """64 MiB of page-locked input takes the chunked three-stream launch path."""
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(16384, 1024, generator=gen)
    plain = torch.empty(16384)
    K.row_sums[16](x, plain, 16384, 1024, 8)
    xp, outp = x.pin_memory(), torch.empty(16384).pin_memory()
    K.row_sums[16](xp, outp, 16384, 1024, 8)
    assert K.row_sums.last_plan.pipeline is not None
    assert torch.equal(outp, plain)
    torch.testing.assert_close(plain, x.sum(1), rtol=1e-5, atol=1e-4)


def test_golden_fixture(golden_dir):
    import os
    import numpy as np
    d = np.load(os.path.join(golden_dir, "elementwise_reduce.npz"))
    x = torch.from_numpy(d["reduce_x"])
    for op, dim, key, exact in ((asc2.reduce_sum, 0, "sum0", False), (asc2.reduce_sum, 1, "sum1", False),
                                (asc2.reduce_max, 0, "max0", True), (asc2.reduce_min, 1, "min1", True),
                                (asc2.reduce_prod, 0, "prod0", False)):
        want = torch.from_numpy(d[key])
        out = torch.zeros_like(want)
        K.reduce_axis[1](x, out, dim, [64, 32], [0, 0], list(want.shape), [0], op, False)
        if exact:
            assert torch.equal(out, want)
        else:
            torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("rows, cols", [(3, 7), (257, 4096), (8, 60000), (4, 70001), (1000, 8), (513, 1000), (300, 2048),
                                        (77, 8192), (33, 16384), (65536, 2048), (50, 3072), (40, 5120), (20, 12288)])
def test_capi_softmax_f16(lib, rows, cols):
    """fp16 rows: every depth of the register kernel (whole 16-byte vectors up to 16384 columns, 256 MiB beyond L2
    included) and the generic path for odd lengths, odd pitches and longer rows (rows staged in shared memory and
    rows too long for it)."""
    gen = torch.Generator(device="cuda").manual_seed(rows + cols)
    pad = 8 if cols % 8 == 0 and rows != 257 else 1      # a pitch of whole vectors keeps the register kernel
    x = (torch.randn(rows, cols + pad, device="cuda", generator=gen) * 3).half()
    out = torch.full_like(x, 9.0)
    rc = lib.asc_cuda_softmax_f16(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, cols, cols + pad, None)
    assert rc == 0, capi.status_string(rc)
    capi.check_device_status(None)
    want = torch.softmax(x[:, :cols].float(), dim=1).half()
    torch.testing.assert_close(out[:, :cols], want, rtol=1e-3, atol=1e-6)
    assert bool((out[:, cols:] == 9.0).all())


# ------------------------------------------------------------------------------- RMS normalisation
@pytest.mark.parametrize("rows, cols, block, blocks", [(64, 256, 8, 4), (4096, 1024, 8, 16), (96, 8192, 1, 3),
                                                       (24, 8, 8, 1)])
def test_rms_norm_rows_kernel(rows, cols, block, blocks):
    gen = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=gen) * 3
    gamma = torch.rand(1, cols, generator=gen) + 0.5
    out = torch.zeros_like(x)
    K.rms_norm_rows[blocks](x, gamma, out, rows, cols, block, 1e-5)
    torch.testing.assert_close(out, golden.rms_norm(x, gamma, 1e-5), rtol=1e-5, atol=1e-6)


def test_rms_norm_1d_and_device_tensors():
    x = torch.randn(1024)
    gamma = torch.rand(1024)
    out = torch.zeros(1024)
    K.rms_norm_1d[1](x, gamma, out, 1024)
    torch.testing.assert_close(out, golden.rms_norm(x, gamma, 1e-6), rtol=1e-5, atol=1e-6)
    xd, gd = torch.randn(512, 2048, device="cuda"), torch.rand(1, 2048, device="cuda")
    od = torch.empty_like(xd)
    K.rms_norm_rows[8](xd, gd, od, 512, 2048, 4, 1e-6)
    torch.testing.assert_close(od.cpu(), golden.rms_norm(xd.cpu(), gd.cpu(), 1e-6), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rows, cols, pad", [(1, 1, 0), (7, 33, 3), (300, 1000, 0), (129, 4096, 4), (33, 8192, 0),
                                             (5, 20000, 0), (9, 16384, 8), (32768, 2048, 0), (50, 3072, 0), (40, 5120, 0),
                                             (30, 6144, 8), (21, 7168, 0), (60, 1280, 0)])
def test_capi_rms_norm(lib, rows, cols, pad):
    """Every register depth of the vector kernel, the two-read kernel (long, ragged or unaligned rows), pitched
    rows, and a 256 MiB matrix (beyond L2); in place as well."""
    gen = torch.Generator(device="cuda").manual_seed(rows * 7 + cols)
    ld = cols + pad
    buf = torch.randn(rows, ld, device="cuda", generator=gen) * 2
    gamma = torch.rand(cols, device="cuda", generator=gen) + 0.25
    out = torch.full((rows, ld), -7.0, device="cuda")
    x = buf[:, :cols]
    rc = lib.asc_cuda_rms_norm_f32(ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(gamma.data_ptr()),
                                   ctypes.c_void_p(out.data_ptr()), rows, cols, ld, 1e-5, None)
    assert rc == 0, capi.status_string(rc)
    capi.check_device_status(None)
    ref = golden.rms_norm(x.double(), gamma.double(), 1e-5) if rows * cols < (1 << 22) else golden.rms_norm(x, gamma, 1e-5)
    torch.testing.assert_close(out[:, :cols], ref.float(), rtol=1e-5, atol=1e-6)
    assert pad == 0 or bool((out[:, cols:] == -7.0).all())          # the pitch padding is untouched
    keep = buf.clone()
    rc = lib.asc_cuda_rms_norm_f32(ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(gamma.data_ptr()),
                                   ctypes.c_void_p(buf.data_ptr()), rows, cols, ld, 1e-5, None)
    assert rc == 0
    assert torch.equal(buf[:, :cols], out[:, :cols]) and torch.equal(buf[:, cols:], keep[:, cols:])


@pytest.mark.parametrize("rows, cols, pad", [(3, 8, 0), (65, 1000, 0), (40, 4096, 8), (17, 8192, 0), (9, 16384, 0),
                                             (11, 1001, 1), (65536, 2048, 0), (50, 3072, 0), (40, 5120, 8), (30, 6144, 0)])
def test_capi_rms_norm_f16(lib, rows, cols, pad):
    """fp16 rows: every register depth, the two-read kernel (long or odd rows), pitched rows, 256 MiB beyond L2."""
    gen = torch.Generator(device="cuda").manual_seed(rows * 5 + cols)
    ld = cols + pad
    buf = (torch.randn(rows, ld, device="cuda", generator=gen) * 2).half()
    gamma = (torch.rand(cols, device="cuda", generator=gen) + 0.25).half()
    out = torch.full((rows, ld), -7.0, device="cuda", dtype=torch.float16)
    rc = lib.asc_cuda_rms_norm_f16(ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(gamma.data_ptr()),
                                   ctypes.c_void_p(out.data_ptr()), rows, cols, ld, 1e-5, None)
    assert rc == 0, capi.status_string(rc)
    capi.check_device_status(None)
    ref = golden.rms_norm(buf[:, :cols], gamma, 1e-5).half()      # fp32 arithmetic, one rounding at the end
    torch.testing.assert_close(out[:, :cols], ref, rtol=1e-3, atol=1e-3)
    assert pad == 0 or bool((out[:, cols:] == -7.0).all())


def test_rms_norm_f16_through_asc2():
    x = (torch.randn(64, 512) * 3).half()
    gamma = (torch.rand(1, 512) + 0.5).half()
    out = torch.zeros_like(x)
    K.rms_norm_rows[4](x, gamma, out, 64, 512, 8, 1e-5)
    torch.testing.assert_close(out, golden.rms_norm(x, gamma, 1e-5).half(), rtol=1e-3, atol=1e-3)


def test_capi_rms_norm_rejects_bad_arguments(lib):
    x = torch.zeros(4, 8, device="cuda")
    p = ctypes.c_void_p(x.data_ptr())
    assert lib.asc_cuda_rms_norm_f32(p, p, p, 4, 8, 4, 1e-5, None) == 1     # invalid argument: pitch < cols
    assert lib.asc_cuda_rms_norm_f32(p, None, p, 4, 8, 8, 1e-5, None) == 1
    assert lib.asc_cuda_rms_norm_f32(None, None, None, 0, 8, 8, 1e-5, None) == 0                   # empty
