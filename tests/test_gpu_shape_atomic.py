"""Shape operations, broadcasts and atomics on the GPU: the reference's operation tests
(python/test/asc2/operations/test_shape_ops.py:10-77, test_atomic_ops.py:13-67: same shapes, dtypes, value
distributions and goldens).  Copies, broadcasts, max / min and integer sums are bit-exact."""
import pytest
import torch

import asc.runtime.config as config
import asc2

import asc2_scripts as K
import eltwise_cases as C

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id):
    config.set_platform(backend, platform, device_id)


@pytest.mark.parametrize("asc_op, torch_op, args, shape, dtype", C.SHAPE_CASES, ids=C.ids)
def test_shape_op(asc_op, torch_op, args, shape, dtype):
    launch, ref = C.shape_case(asc_op, torch_op, args, shape, dtype)
    z = launch()
    torch.testing.assert_close(z, ref, atol=1e-3, rtol=1e-3)
    assert torch.equal(z, ref)


@pytest.mark.parametrize("shape", ([32], [3, 32]), ids=str)
@pytest.mark.parametrize("dtype", (torch.float16, torch.float32, torch.int16, torch.int32), ids=str)
def test_broadcast_dup(shape, dtype):
    out = torch.zeros(shape, dtype=dtype)
    K.broadcast_dup[1](out, tuple(out.size()), [0] * out.dim())
    torch.testing.assert_close(out, torch.full_like(out, 777), atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("asc_op, torch_op, dtype", C.ATOMIC_CASES, ids=C.ids)
def test_atomic_op(asc_op, torch_op, dtype):
    launch, expected = C.atomic_case(asc_op, torch_op, dtype)
    z = launch()
    torch.testing.assert_close(z, expected, atol=1e-3, rtol=1e-3)
    if asc_op is not asc2.atomic_add or dtype != torch.float32:
        assert torch.equal(z, expected)


def test_atomic_add_many_blocks():
    launch, expected = C.atomic_case(asc2.atomic_add, torch.add, torch.int32, cores=64, size=64 * 256)
    assert torch.equal(launch(), expected)


@pytest.mark.parametrize("rows, cols, rows_per_tile, cores", [(4096, 1024, 8, 16), (1000, 256, 8, 5)])
def test_bias_row_broadcast(rows, cols, rows_per_tile, cores):
    gen = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, cols, generator=gen)
    b = torch.randn(1, cols, generator=gen)
    out = torch.full_like(x, -3.0)
    K.add_row_bias[cores](x, b, out, rows, cols, rows_per_tile)
    assert torch.equal(out, torch.relu(x + b))


def test_concat_rows_and_nested_concat():
    """asc2.concat joins tiles along the first dimension; the stored parts land at their row offsets."""
    gen = torch.Generator().manual_seed(11)
    a, b = torch.randn(32, 64, generator=gen), torch.randn(32, 64, generator=gen)
    out = torch.full((64, 64), -1.0)
    K.concat_rows[4](a, b, out, 32, 32, 64, 8)
    ref = torch.cat([torch.cat([2 * a[i:i + 8], b[i:i + 8]]) for i in range(0, 32, 8)])
    assert torch.equal(out, ref)
    x, y = torch.randn(64, generator=gen), torch.randn(64, generator=gen)
    flat = torch.zeros(192)
    K.concat_1d[1](x, y, flat, 64)
    assert torch.equal(flat, torch.cat([x, y, x + y]))
