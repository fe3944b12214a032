"""Tile loads and stores anywhere in a tensor, on the GPU: the reference's memory-operation tests
(python/test/asc2/operations/test_memory_ops.py: same shapes, tile ids / offsets, goldens) and the 2-D
window entry point at sizes beyond L2.  Additions are bit-exact; untouched elements must stay untouched."""
import ctypes

import pytest
import torch

import asc.runtime.config as config

import asc2_scripts as K
import eltwise_cases as C
from oracle import eltwise as E
from pyasc_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id):
    config.set_platform(backend, platform, device_id)


@pytest.mark.parametrize("case", C.MEMORY_CASES, ids=str)
def test_load_store(case):
    launch, expected, _ = C.memory_case(*case)
    z = launch()
    torch.testing.assert_close(z, expected, atol=1e-3, rtol=1e-3)
    assert torch.equal(z, expected)


@pytest.mark.parametrize("tensor_shape, offsets", [((16, ), (0, )), ((16, ), (7, )), ((16, 16), (0, 0)), ((16, 16), (7, 7))],
                         ids=str)
def test_store_1elem_tile(tensor_shape, offsets):
    x = torch.randn(tensor_shape, dtype=torch.float32)
    y = torch.zeros_like(x)
    K.copy_1elem[1](x, y, tensor_shape, offsets)
    expected = torch.zeros_like(x)
    expected[offsets] = x[offsets]
    assert torch.equal(y, expected)


@pytest.mark.parametrize("rows, cols, tile_r, tile_c, cores", [(1000, 1000, 64, 128, 16), (130, 70, 32, 32, 3),
                                                               (4096, 4096, 128, 256, 148)])
def test_2d_tile_grid_kernel(rows, cols, tile_r, tile_c, cores):
    gen = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=gen)
    out = torch.full_like(x, -7.0)
    K.scale_2d_tiles[cores](x, out, rows, cols, 0.5, tile_r, tile_c)
    torch.testing.assert_close(out, torch.tanh(x * 0.5), rtol=2e-6, atol=1e-6)


# ------------------------------------------------------------------------------- C ABI
@pytest.fixture(scope="module")
def lib():
    torch.cuda.set_device(0)
    return capi.load()


@pytest.mark.parametrize("dtype, out_type, round_op", [(torch.float32, 0, None), (torch.bfloat16, 2, 34)], ids=str)
@pytest.mark.parametrize("R, C_, r0, c0, rows, cols", [
    (64, 64, 3, 5, 7, 9),                    # odd origin and size: scalar path
    (512, 1024, 128, 256, 128, 512),         # aligned: quads
    (8192, 8192, 4096, 1024, 4096, 6144),    # 96 MiB fp32 window inside a 256 MiB matrix
    (300, 1000, 0, 0, 300, 1000),            # the whole matrix (ld == cols: flat)
], ids=str)
def test_window_program_bit_exact_and_confined(lib, dtype, out_type, round_op, R, C_, r0, c0, rows, cols):
    gen = torch.Generator(device="cuda").manual_seed(R + c0)
    x = (torch.rand(R, C_, device="cuda", generator=gen) * 4 - 2).to(dtype)
    y = (torch.rand(R, C_, device="cuda", generator=gen) * 4 - 2).to(dtype)
    out = torch.full((R, C_), 3.0, device="cuda", dtype=dtype)
    ops = [0, 0, 4] + ([round_op] if round_op else []) + [2 | 0x100] + ([round_op] if round_op else [])
    args = [0, 1, 0] + ([0] if round_op else []) + [int(torch.tensor(0.25).view(torch.int32))] + ([0] if round_op else [])
    es = x.element_size()
    first = (r0 * C_ + c0) * es
    ops_a, args_a = (ctypes.c_int32 * len(ops))(*ops), (ctypes.c_int32 * len(ops))(*args)
    ins = (ctypes.c_void_p * 2)(x.data_ptr() + first, y.data_ptr() + first)
    types = (ctypes.c_int32 * 2)(out_type, out_type)
    lds = (ctypes.c_int64 * 3)(C_, C_, C_)
    rc = lib.asc_cuda_eltwise_program_2d(ops_a, args_a, len(ops), ins, types, 2, ctypes.c_void_p(out.data_ptr() + first),
                                         out_type, rows, cols, lds, None)
    assert rc == 0, capi.status_string(rc)
    capi.check_device_status(None)
    want = torch.full((R, C_), 3.0, dtype=dtype)
    xw, yw = x[r0:r0 + rows, c0:c0 + cols].cpu().reshape(-1), y[r0:r0 + rows, c0:c0 + cols].cpu().reshape(-1)
    want[r0:r0 + rows, c0:c0 + cols] = E.run_program(ops, args, [xw, yw], out_type).reshape(rows, cols)
    assert torch.equal(out.cpu(), want)


def test_broadcast_row_and_mixed_pitches(lib):
    """out[r, c] = x[r, c] * b[c] + y[r, c]: x from a wider matrix, y contiguous, b one row (pitch 0)."""
    gen = torch.Generator(device="cuda").manual_seed(9)
    rows, cols = 3000, 1024
    x = torch.randn(rows, cols + 64, device="cuda", generator=gen)
    y = torch.randn(rows, cols, device="cuda", generator=gen)
    b = torch.randn(cols, device="cuda", generator=gen)
    out = torch.full((rows, cols + 8), 5.0, device="cuda")
    ops, args = [0, 0, 4, 0, 2], [0, 1, 0, 2, 0]
    ops_a, args_a = (ctypes.c_int32 * 5)(*ops), (ctypes.c_int32 * 5)(*args)
    ins = (ctypes.c_void_p * 3)(x.data_ptr(), b.data_ptr(), y.data_ptr())
    types = (ctypes.c_int32 * 3)(0, 0, 0)
    lds = (ctypes.c_int64 * 4)(cols + 64, 0, cols, cols + 8)
    rc = lib.asc_cuda_eltwise_program_2d(ops_a, args_a, 5, ins, types, 3, ctypes.c_void_p(out.data_ptr()), 0, rows, cols,
                                         lds, None)
    assert rc == 0, capi.status_string(rc)
    capi.check_device_status(None)
    assert torch.equal(out[:, :cols], x[:, :cols] * b + y) and bool((out[:, cols:] == 5.0).all())


def test_window_program_rejections(lib):
    x = torch.zeros(16, 16, device="cuda")
    ops_a, args_a = (ctypes.c_int32 * 1)(0), (ctypes.c_int32 * 1)(0)
    ins, types = (ctypes.c_void_p * 1)(x.data_ptr()), (ctypes.c_int32 * 1)(0)
    out = ctypes.c_void_p(x.data_ptr())

    def call(rows, cols, pitches):
        lds = (ctypes.c_int64 * 2)(*pitches)
        return lib.asc_cuda_eltwise_program_2d(ops_a, args_a, 1, ins, types, 1, out, 0, rows, cols, lds, None)
    assert call(4, 8, (4, 8)) == 1                       # an input pitch smaller than the row (and not 0)
    assert call(4, 8, (8, 0)) == 1                       # the output cannot be a broadcast row
    assert call(-1, 8, (8, 8)) == 1
    assert call(1 << 20, 1 << 12, (1 << 13, 1 << 13)) == 6
    assert call(0, 8, (16, 16)) == 0                     # empty


@pytest.mark.parametrize("dtype", [torch.int8, torch.uint8, torch.float64, torch.int64], ids=str)
def test_copy_of_tiles_of_any_element_type(dtype):
    """asc2.store(asc2.load(...)) moves bytes: 8-bit and 64-bit tiles, windows of matrices of different widths."""
    import asc2_scripts as K
    gen = torch.Generator().manual_seed(3)
    x = torch.randint(-100, 100, (64, 256), generator=gen).to(dtype)
    out = torch.full((64, 512), 7, dtype=dtype)
    K.copy_window[4](x, out, 64, 256, 512, 128, 64, 32, 8)
    want = torch.full((64, 512), 7, dtype=dtype)
    want[:, 32:160] = x[:, 64:192]
    assert torch.equal(out, want)
    # whole matrices, and a window whose byte offsets are not multiples of 16
    y = torch.randint(-100, 100, (64, 128), generator=gen).to(dtype)
    out2 = torch.zeros_like(y)
    K.copy_window[4](y, out2, 64, 128, 128, 128, 0, 0, 8)
    assert torch.equal(out2, y)
    if dtype in (torch.int8, torch.uint8):
        out3 = torch.full((64, 512), 7, dtype=dtype)
        K.copy_window[4](x, out3, 64, 256, 512, 96, 32, 32, 8)
        want3 = torch.full((64, 512), 7, dtype=dtype)
        want3[:, 32:128] = x[:, 32:128]
        assert torch.equal(out3, want3)


def test_capi_copy_2d_vector_and_byte_paths():
    lib = capi.load()
    gen = torch.Generator().manual_seed(4)
    src = torch.randint(0, 255, (300, 1000), generator=gen).to(torch.uint8).cuda()
    P = lambda t, off=0: ctypes.c_void_p(t.data_ptr() + off)
    for (rows, row_bytes, s_off, d_off) in ((300, 1000, 0, 0), (257, 333, 7, 5), (64, 512, 16, 32), (1, 1, 999, 3), (0, 10, 0, 0)):
        dst = torch.full((300, 1200), 9, dtype=torch.uint8, device="cuda")
        rc = lib.asc_cuda_copy_2d(P(dst, d_off), P(src, s_off), rows, row_bytes, 1200, 1000, None)
        assert rc == 0, capi.status_string(rc)
        capi.check_device_status(None)
        want = torch.full((300, 1200), 9, dtype=torch.uint8)
        flat_s, flat_d = src.cpu().reshape(-1), want.reshape(-1)
        for r in range(rows):
            flat_d[d_off + r * 1200:d_off + r * 1200 + row_bytes] = flat_s[s_off + r * 1000:s_off + r * 1000 + row_bytes]
        assert torch.equal(dst.cpu(), want), (rows, row_bytes, s_off, d_off)
    dst = torch.zeros(16, dtype=torch.uint8, device="cuda")
    assert lib.asc_cuda_copy_2d(P(dst), P(src), 2, 16, 8, 1000, None) == 1          # pitch shorter than a row
    assert lib.asc_cuda_copy_2d(None, P(src), 2, 8, 8, 1000, None) == 1
