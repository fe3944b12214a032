"""Inputs, launches and torch goldens of the elementwise kernels, shared by the CPU tests (compiled
program evaluated by the CPU oracle) and the GPU tests (the same launches run on the device).  Cases
and value distributions follow python/test/asc2/operations/test_{binary_ops,unary_ops,where}.py and
python/test/asc2/kernels/test_{leaky_relu,gelu}.py."""
import math

import torch

import asc
import asc2

import asc2_scripts as K

BINARY_OPS = [
    (asc2.add, torch.add, [K.VV, K.VS, K.SV], [torch.bfloat16, torch.float32, torch.int32]),
    (asc2.div, torch.div, [K.VV, K.VS, K.SV], [torch.float32]),
    (asc2.mul, torch.mul, [K.VV, K.VS, K.SV], [torch.bfloat16, torch.float32, torch.int32]),
    (asc2.sub, torch.sub, [K.VV, K.VS, K.SV], [torch.bfloat16, torch.float32, torch.int32]),
    (asc2.left_shift, torch.bitwise_left_shift, [K.VS], [torch.int32]),
    (asc2.right_shift, torch.bitwise_right_shift, [K.VS], [torch.int32]),
    (asc2.maximum, torch.maximum, [K.VV, K.VS, K.SV], [torch.bfloat16, torch.float32, torch.int32]),
    (asc2.minimum, torch.minimum, [K.VV, K.VS, K.SV], [torch.bfloat16, torch.float32, torch.int32]),
]
BINARY_CASES = [(a, t, f, d) for a, t, fmts, dtypes in BINARY_OPS for f in fmts for d in dtypes]

UNARY_OPS = [
    (asc2.abs, torch.abs), (asc2.ceil, torch.ceil), (asc2.cos, torch.cos), (asc2.cosh, torch.cosh),
    (asc2.erf, torch.erf), (asc2.exp, torch.exp), (asc2.exp2, torch.exp2), (asc2.floor, torch.floor),
    (asc2.log, torch.log), (asc2.negative, torch.neg), (asc2.relu, torch.relu), (asc2.rsqrt, torch.rsqrt),
    (asc2.sin, torch.sin), (asc2.sinh, torch.sinh), (asc2.sqrt, torch.sqrt), (asc2.tan, torch.tan),
    (asc2.tanh, torch.tanh),
]

COMPARE_OPS = [(asc2.equal, torch.eq), (asc2.not_equal, torch.ne), (asc2.greater, torch.gt),
               (asc2.greater_equal, torch.ge), (asc2.less, torch.lt), (asc2.less_equal, torch.le)]
WHERE_DTYPES = [torch.float16, torch.bfloat16, torch.float32, torch.int16, torch.int32]


def ids(obj) -> str:
    return obj.__name__ if callable(obj) else str(obj)


def binary_case(asc_op, torch_op, fmt, dtype):
    """Returns (launch, golden, runtime_args): ``launch()`` runs the kernel and returns the output
    tensor; ``runtime_args`` are the kernel's run-time arguments in order."""
    size = 32
    gen = torch.Generator().manual_seed(2026)

    def operand(is_vector: bool):
        if not is_vector:
            return torch.tensor(2, dtype=dtype)
        if dtype.is_floating_point:
            return torch.randn((size, ), dtype=dtype, generator=gen).clamp(1, 100)
        return torch.randint(1, 100, (size, ), dtype=dtype, generator=gen)

    x = operand(fmt in (K.VV, K.VS))
    y = operand(fmt in (K.VV, K.SV))
    z = torch.zeros(size, dtype=dtype)

    def launch():
        K.binary_op[1](x, y, z, size, fmt, asc_op)
        return z

    return launch, torch_op(x, y), [x, y, z]


def unary_case(asc_op, torch_op):
    gen = torch.Generator().manual_seed(2026)
    x = torch.randn((32, ), dtype=torch.float32, generator=gen).clamp(1, 100)
    z = torch.zeros(32, dtype=torch.float32)

    def launch():
        K.unary_op[1](x, z, 32, asc_op)
        return z

    return launch, torch_op(x), [x, z]


def _where_tensor(dtype, gen):
    if dtype.is_floating_point:
        return torch.rand(K.WHERE_SIZE, dtype=dtype, generator=gen)
    return torch.randint(-100, 100, (K.WHERE_SIZE, ), dtype=dtype, generator=gen)


def where_case(asc_op, torch_op, dtype, scalar: bool):
    gen = torch.Generator().manual_seed(2026)
    x = _where_tensor(dtype, gen)
    result = torch.zeros_like(x)
    if scalar:
        y = torch.tensor(0 if not dtype.is_floating_point else 0.5, dtype=dtype)
        golden = torch.where(torch_op(x, y), torch.tensor(0, dtype=dtype), torch.tensor(1, dtype=dtype))

        def launch():
            K.where_scalar_op[1](x, y, result, asc_op)
            return result
    else:
        y = _where_tensor(dtype, gen)
        y[::5] = x[::5]          # make the equality branches non-trivial
        golden = torch.where(torch_op(x, y), x, y)

        def launch():
            K.where_op[1](x, y, result, asc_op)
            return result
    return launch, golden, [x, y, result]


def leaky_relu_case(size=8192, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(2026)
    x = (torch.rand(size, generator=gen) * 10.0 - 5.0).to(dtype)
    alpha = torch.tensor(0.1, dtype=dtype)
    out = torch.empty_like(x)
    core_num, tile_size = 16, 128
    num_tiles = asc.ceildiv(size, tile_size)

    def launch():
        K.leaky_relu[core_num](x, alpha, out, size, tile_size, asc.ceildiv(num_tiles, core_num))
        return out

    return launch, torch.where(x >= 0, x, x * alpha), [x, alpha, out, size]


def gelu_torch(x: torch.Tensor, approximate: bool):
    if approximate:
        return 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * torch.pow(x, 3))))
    return 0.5 * x * (1 + torch.erf(x / math.sqrt(2)))


def gelu_case(approximate: bool, rows=30, cols=1024):
    gen = torch.Generator().manual_seed(2026)
    x = torch.rand((rows, cols), dtype=torch.float32, generator=gen)
    out = torch.empty_like(x)

    def launch():
        K.gelu[16](x, out, rows, cols, cols, approximate)
        return out

    return launch, gelu_torch(x, approximate), [x, out]


# (dim, tensor_shape, tile_shape, tile_id, offsets, is_static): python/test/asc2/operations/test_memory_ops.py:10-59
MEMORY_CASES = [
    (1, [64], [16], [0], None, True), (1, [64], [16], [3], None, True),
    (2, [128, 128], [32, 32], [0, 0], None, True), (2, [128, 128], [32, 32], [3, 3], None, True),
    (2, [1024, 512], [128, 64], [1, 2], None, True), (1, [37], [8], [3], None, True),
    (2, [123, 456], [13, 16], [2, 5], None, True),
    (1, [64], [16], None, [0], True), (1, [64], [16], None, [48], True),
    (2, [128, 128], [32, 32], None, [0, 0], True), (2, [128, 128], [32, 32], None, [96, 64], True),
    (2, [1024, 512], [128, 64], None, [256, 128], True), (1, [53], [16], None, [22], True),
    (2, [257, 511], [19, 24], None, [40, 64], True),
    (1, [32], [8], [1], None, False), (1, [32], [8], [3], None, False),
    (2, [16, 2048], [4, 512], [0, 3], None, False), (2, [16, 2048], [8, 256], [1, 7], None, False),
    (2, [512, 512], [64, 64], [4, 4], None, False), (1, [99], [16], [5], None, False),
    (2, [1000, 1000], [33, 40], [1, 1], None, False),
    (1, [32], [8], None, [16], False), (1, [32], [8], None, [24], False),
    (2, [16, 2048], [4, 512], None, [8, 1024], False), (2, [16, 2048], [12, 1024], None, [4, 0], False),
    (2, [512, 512], [64, 64], None, [128, 256], False), (1, [77], [24], None, [48], False),
    (2, [150, 300], [21, 40], None, [10, 20], False),
    (1, [32], None, None, [0], True), (2, [32, 32], None, None, [0, 0], True),
    (1, [1024], None, None, [0], True), (2, [512, 512], None, None, [0, 0], True),
]


def memory_case(dim, tensor_shape, tile_shape, tile_id, offsets, is_static):
    """Returns (launch, expected): z = x + y inside the addressed tile (or element), zero elsewhere."""
    gen = torch.Generator().manual_seed(2026)
    x, y = [torch.randn(tensor_shape, generator=gen) for _ in range(2)]
    z = torch.zeros(tensor_shape, dtype=torch.float32)

    def launch():
        if is_static:
            if tile_shape is None:
                K.add_scalar[1](x, y, z, tensor_shape, offsets)
            else:
                K.add_static[1](x, y, z, tensor_shape, tile_shape, tile_id, offsets)
        elif dim == 1:
            K.add_dynamic_1d[1](x, y, z, tensor_shape[0], tile_shape, tile_id, offsets)
        else:
            K.add_dynamic_2d[1](x, y, z, tensor_shape[0], tensor_shape[1], tile_shape, tile_id, offsets)
        return z

    actual = [i * s for i, s in zip(tile_id, tile_shape)] if tile_id is not None else offsets
    if tile_shape is not None:
        slices = tuple(slice(off, off + size) for off, size in zip(actual, tile_shape))
    else:
        slices = tuple(actual)
    expected = torch.zeros_like(z)
    expected[slices] = x[slices] + y[slices]
    kernel = K.add_scalar if tile_shape is None else K.add_static if is_static else \
        K.add_dynamic_1d if dim == 1 else K.add_dynamic_2d
    return launch, expected, kernel


# (asc2 op, torch op, op arguments, input shape): python/test/asc2/operations/test_shape_ops.py:10-18
SHAPE_OPS = [
    (asc2.broadcast_to, torch.broadcast_to, [4, 32], [1, 32]), (asc2.broadcast_to, torch.broadcast_to, [50, 32], [1, 32]),
    (asc2.reshape, torch.reshape, [64], [2, 32]), (asc2.reshape, torch.reshape, [4, 16], [64]),
    (asc2.ravel, torch.ravel, [], [2, 32]), (asc2.expand_dims, torch.unsqueeze, [0], [32]),
    (asc2.squeeze, torch.squeeze, [0], [1, 32]),
]
SHAPE_CASES = [(a, t, args, shape, d) for a, t, args, shape in SHAPE_OPS for d in (torch.float16, torch.float32, torch.int32)]


def shape_case(asc_op, torch_op, args, shape, dtype):
    gen = torch.Generator().manual_seed(2026)

    def create_input(tensor_shape):
        if dtype.is_floating_point:
            return torch.randn(tuple(tensor_shape), dtype=dtype, generator=gen).clamp(1, 100)
        return torch.randint(1, 100, tuple(tensor_shape), dtype=dtype, generator=gen)

    x = create_input(shape)
    if asc_op in (asc2.expand_dims, asc2.squeeze):
        ref_z = torch_op(x, dim=args[0])
    elif not args:
        ref_z = torch_op(x)
    else:
        ref_z = torch_op(x, args)
    z = create_input(ref_z.shape)

    def launch():
        K.shape_op[1](x, z, tuple(x.shape), tuple(ref_z.shape), (0, ) * x.dim(), (0, ) * ref_z.dim(), asc_op, args)
        return z

    return launch, ref_z.contiguous()


ATOMIC_CASES = [(a, t, d) for a, t in ((asc2.atomic_add, torch.add), (asc2.atomic_max, torch.maximum),
                                       (asc2.atomic_min, torch.minimum))
                for d in (torch.float32, torch.float16, torch.int32)]


def atomic_case(asc_op, torch_op, dtype, cores=4, size=128):
    gen = torch.Generator().manual_seed(2026)

    def create_input(shape):
        if dtype == torch.float32:
            return torch.randn(tuple(shape), dtype=dtype, generator=gen).clamp(1, 100)
        return torch.randint(1, 100, tuple(shape), generator=gen).to(dtype)

    tile_length = size // cores
    x = create_input([size])
    z = create_input([tile_length])
    expected = z.clone()
    for i in range(cores):
        expected = torch_op(expected, x[i * tile_length:(i + 1) * tile_length] + 10)

    def launch():
        K.atomic_op[cores](x, z, [size], tile_length, asc_op)
        return z

    return launch, expected
