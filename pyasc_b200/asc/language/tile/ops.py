"""The asc2 tile operations, recorded instead of lowered
(reference: python/asc/language/tile/{memory,binary,unary,reduction,creation,shape,indexing,atomic,
prog_model}_ops.py).  Argument checks and result shapes/dtypes follow the reference; each call
appends one node to the active trace."""
from __future__ import annotations

import contextlib

import math
from typing import Any, Iterable, List, Optional, Tuple, Union

from ..core.dtype import DataType, KnownTypes as KT
from ..core.ir_value import PlainValue
from . import trace
from .tensor import Tensor
from .tile import BinaryOperandTypeError, Tile, TileLocation
from .utils import check_data_alignment, infer_dtype, infer_shape, verify_shape

Numeric = (bool, int, float)


def _scalar(v: Any) -> PlainValue:
    return PlainValue.wrap(v)


def _offsets(values: Iterable) -> Tuple[PlainValue, ...]:
    return tuple(_scalar(v) for v in values)


def _infer_offsets(rank_shape, shape, tile_id, offsets) -> Tuple[PlainValue, ...]:
    shape = tuple(shape)
    if len(rank_shape) != len(shape):
        raise RuntimeError("rank of 'tensor_shape' must match rank of 'shape'")
    if tile_id is not None:
        return _offsets(idx * size for idx, size in zip(tile_id, shape))
    offs = _offsets(offsets)
    if len(offs) != len(shape):
        raise RuntimeError("number of 'offsets' must match rank of 'shape'")
    return offs


# ------------------------------------------------------------------------------------------------
# memory
# ------------------------------------------------------------------------------------------------
def load(tensor: Tensor, shape: Optional[Iterable[int]] = None, *, tile_id: Optional[Iterable] = None,
         offsets: Optional[Iterable] = None, location: TileLocation = TileLocation.UB, pad_value: Any = 0):
    if (tile_id is None) == (offsets is None):
        raise ValueError("Exactly one of 'tile_id' or 'offsets' must be provided")
    ctx = trace.current()
    if shape is None:
        node = ctx.node("load_scalar", tensor, offsets=_offsets(offsets))
        return PlainValue("tile_scalar", (node, ), tensor.dtype)
    shape = verify_shape(shape)
    check_data_alignment(shape, tensor.dtype)
    offs = _infer_offsets(tensor.shape, shape, tile_id, offsets)
    node = ctx.node("load", tensor, offsets=offs, shape=shape, pad_value=pad_value)
    return Tile(shape, tensor.dtype, node, location)


def copy(tile: Tile, shape: Optional[Iterable[int]] = None, *, offsets: Optional[Iterable] = None,
         location: TileLocation = TileLocation.UB) -> Tile:
    if shape is None:
        shape = tile.shape
    if offsets is None:
        offsets = (0, ) * len(tile.shape)
    shape = verify_shape(shape)
    check_data_alignment(shape, tile.dtype)
    offs = _infer_offsets(tile.shape, shape, None, offsets)
    node = trace.current().node("copy", tile, offsets=offs, shape=shape, location=location)
    return Tile(shape, tile.dtype, node, location)


def store(value: Any, tensor: Tensor, *, tile_id: Optional[Iterable] = None, offsets: Optional[Iterable] = None) -> None:
    ctx = trace.current()
    scalar_store = not isinstance(value, Tile) or value.size == 1
    if scalar_store:
        if tile_id is not None:
            raise ValueError("'tile_id' argument cannot be used when storing a scalar value or a tile with 1 element")
        if offsets is None:
            raise ValueError("'offsets' argument must be provided")
        ctx.effect("store_scalar", value, tensor, offsets=_offsets(offsets))
        return
    if (tile_id is None) == (offsets is None):
        raise ValueError("Exactly one of 'tile_id' or 'offsets' must be provided")
    check_data_alignment(value.shape, value.dtype)
    offs = _infer_offsets(tensor.shape, value.shape, tile_id, offsets)
    ctx.effect("store", value, tensor, offsets=offs)


# ------------------------------------------------------------------------------------------------
# binary / compare
# ------------------------------------------------------------------------------------------------
def _binary(op: str, lhs: Any, rhs: Any) -> Tile:
    if not isinstance(lhs, Tile) and not isinstance(rhs, Tile):
        raise BinaryOperandTypeError(f"At least one operand of '{op}' must be a tile")
    for v in (lhs, rhs):
        if not isinstance(v, (Tile, PlainValue) + Numeric):
            raise BinaryOperandTypeError(f"Unsupported operand for '{op}': {type(v).__name__}")
    dtype = infer_dtype(lhs, rhs)
    shape = infer_shape(lhs, rhs)
    a = lhs if isinstance(lhs, Tile) else _scalar(lhs)
    b = rhs if isinstance(rhs, Tile) else _scalar(rhs)
    return _masked(Tile(shape, dtype, trace.current().node("binary", a, b, op=op)))


def _compare(mode: str, lhs: Any, rhs: Any) -> Tile:
    if not isinstance(lhs, Tile):
        raise BinaryOperandTypeError("The first operand of a comparison must be a tile")
    shape = infer_shape(lhs, rhs)
    b = rhs if isinstance(rhs, Tile) else _scalar(rhs)
    return Tile(shape, KT.bool_, trace.current().node("compare", lhs, b, mode=mode))


def add(input, other): return _binary("add", input, other)
def sub(input, other): return _binary("sub", input, other)
def mul(input, other): return _binary("mul", input, other)
def div(input, other): return _binary("div", input, other)
def maximum(input, other): return _binary("max", input, other)
def minimum(input, other): return _binary("min", input, other)
def equal(input, other): return _compare("eq", input, other)
def not_equal(input, other): return _compare("ne", input, other)
def greater(input, other): return _compare("gt", input, other)
def greater_equal(input, other): return _compare("ge", input, other)
def less(input, other): return _compare("lt", input, other)
def less_equal(input, other): return _compare("le", input, other)


def _shift(op: str, input: Tile, other: Any) -> Tile:
    if not isinstance(input, Tile) or not input.dtype.is_int():
        raise RuntimeError("Shift operations require an integer tile")
    return Tile(input.shape, input.dtype, trace.current().node("binary", input, _scalar(other), op=op))


def left_shift(input, other): return _shift("shl", input, other)
def right_shift(input, other): return _shift("shr", input, other)


def verify_matmul_arguments(input: Tile, other: Tile, trans_b: bool = False) -> None:
    if not isinstance(input, Tile) or not isinstance(other, Tile):
        raise BinaryOperandTypeError(f"Input operands must be tiles, got {type(input)} and {type(other)}")
    if input.dtype != other.dtype:
        raise RuntimeError(f"Input tiles must have the same types, got {input.dtype} and {other.dtype}")
    # int8 operands are an extension of the CUDA platform (the reference accepts floats only,
    # python/asc/language/tile/utils.py:134)
    if input.dtype not in (KT.float32, KT.float16, KT.bfloat16, KT.int8):
        raise RuntimeError(f"Input tiles have unsupported types: {input.dtype}")
    if len(input.shape) != 2 or len(other.shape) != 2:
        raise RuntimeError(f"Input tiles must have two dims, got {len(input.shape)} and {len(other.shape)}")
    inner = other.shape[1] if trans_b else other.shape[0]
    if input.shape[1] != inner:
        raise RuntimeError(f"Input tiles have incompatible shapes: {input.shape}, {other.shape}")


def matmul(input: Tile, other: Tile, trans_b: bool = False) -> Tile:
    """``input @ other`` with fp32 (int32 for int8 operands) result in the accumulator.
    ``trans_b=True`` (CUDA platform extension) multiplies by ``other`` transposed, so that a
    row-major ``[keys, head_dim]`` tile can serve as the right operand of ``Q @ K^T``."""
    verify_matmul_arguments(input, other, trans_b)
    n = other.shape[0] if trans_b else other.shape[1]
    out_dtype = KT.int32 if input.dtype == KT.int8 else KT.float32
    node = trace.current().node("matmul", input, other, trans_b=bool(trans_b))
    return Tile((input.shape[0], n), out_dtype, node, TileLocation.L0C)


def matmul_acc(input: Tile, other: Tile, acc: Tile) -> None:
    verify_matmul_arguments(input, other)
    if not isinstance(acc, Tile) or acc.shape != (input.shape[0], other.shape[1]):
        raise RuntimeError("Accumulator tile has an incompatible shape")
    ctx = trace.current()
    # the accumulator is updated in place: its defining node becomes "previous value + a @ b"
    acc.node = ctx.node("acc", acc.node, input, other)
    ctx.effect("matmul_acc", input, other, acc)


# ------------------------------------------------------------------------------------------------
# unary
# ------------------------------------------------------------------------------------------------
_SCALAR_MATH = {"sqrt": math.sqrt, "exp": math.exp, "erf": math.erf}


def _unary(op: str, input: Any, float_only: bool = True):
    if not isinstance(input, Tile):
        if op in _SCALAR_MATH and isinstance(input, Numeric):
            return PlainValue.const(float(_SCALAR_MATH[op](input)))
        if op in _SCALAR_MATH and isinstance(input, PlainValue) and input.is_const:
            return PlainValue.const(float(_SCALAR_MATH[op](input.value)))
        raise RuntimeError(f"'{op}' expects a tile, got {type(input).__name__}")
    if float_only and not input.dtype.is_float():
        raise RuntimeError(f"'{op}' supports floating-point tiles only, got {input.dtype}")
    return _masked(Tile(input.shape, input.dtype, trace.current().node("unary", input, op=op), input.location))


def cos(input): return _unary("cos", input)
def sin(input): return _unary("sin", input)
def tan(input): return _unary("tan", input)
def sinh(input): return _unary("sinh", input)
def cosh(input): return _unary("cosh", input)
def tanh(input): return _unary("tanh", input)
def erf(input): return _unary("erf", input)
def exp(input): return _unary("exp", input)
def exp2(input): return _unary("exp2", input)
def log(input): return _unary("log", input)
def log2(input): return _unary("log2", input)
def floor(input): return _unary("floor", input)
def ceil(input): return _unary("ceil", input)
def abs(input): return _unary("abs", input, float_only=False)  # noqa: A001
def rsqrt(input): return _unary("rsqrt", input)
def sqrt(input): return _unary("sqrt", input)
def relu(input): return _unary("relu", input, float_only=False)
def negative(input): return _unary("neg", input, float_only=False)


def softmax(input: Tile) -> Tile:
    if not isinstance(input, Tile):
        raise RuntimeError("'softmax' expects a tile")
    if input.dtype not in (KT.float32, KT.float16):
        raise RuntimeError(f"'softmax' supports float32 and float16 tiles, got {input.dtype}")
    if len(input.shape) > 2:
        raise RuntimeError("'softmax' supports 1-D and 2-D tiles")
    return Tile(input.shape, input.dtype, trace.current().node("softmax", input))


def rms_norm(input: Tile, gamma: Tile, epsilon: Any) -> Tile:
    if not isinstance(input, Tile) or not isinstance(gamma, Tile):
        raise RuntimeError("'rms_norm' expects tiles")
    if input.dtype not in (KT.float32, KT.float16) or gamma.dtype != input.dtype:
        raise RuntimeError(f"'rms_norm' supports float32 and float16 tiles of one type, got {input.dtype} and {gamma.dtype}")
    if len(input.shape) > 2:
        raise RuntimeError("'rms_norm' supports 1-D and 2-D tiles")
    return Tile(input.shape, input.dtype, trace.current().node("rms_norm", input, gamma, _scalar(epsilon)))


def cast(input: Tile, dtype: DataType) -> Tile:
    if input.dtype == dtype:
        return input
    from_i, from_f = input.dtype.is_signed(), input.dtype.is_float()
    to_i, to_f = dtype.is_signed(), dtype.is_float()
    ok = False
    if (from_f or from_i) and (to_f or to_i):
        if input.dtype.bitwidth == dtype.bitwidth and ((from_f and to_i) or (from_i and to_f)):
            ok = True
        elif (input.dtype.bitwidth != dtype.bitwidth and (from_i and to_i)) or (from_f and to_f):
            ok = True
    if not ok:
        raise RuntimeError(f"Cast from {input.dtype} to {dtype} is not supported")
    return Tile(input.shape, dtype, trace.current().node("cast", input, dtype=dtype), input.location)


# ------------------------------------------------------------------------------------------------
# reductions
# ------------------------------------------------------------------------------------------------
def _reduce(kind: str, input: Tile, dims: Tuple[int, ...], keep_dims: bool):
    if not isinstance(input, Tile):
        raise RuntimeError(f"'reduce_{kind}' expects a tile")
    ctx = trace.current()
    if not dims:
        node = ctx.node("reduce", input, kind=kind, dims=(), keep_dims=False)
        return PlainValue("tile_scalar", (node, ), input.dtype)
    rank = len(input.shape)
    norm = tuple(sorted(d + rank if d < 0 else d for d in dims))
    if any(d < 0 or d >= rank for d in norm) or len(set(norm)) != len(norm):
        raise RuntimeError(f"Invalid reduction dims {dims} for a tile of rank {rank}")
    shape = [1 if i in norm else s for i, s in enumerate(input.shape)] if keep_dims else \
        [s for i, s in enumerate(input.shape) if i not in norm]
    if not shape:
        shape = [1]
    node = ctx.node("reduce", input, kind=kind, dims=norm, keep_dims=keep_dims)
    return Tile(tuple(shape), input.dtype, node)


def reduce_sum(input, *dims, keep_dims=False): return _reduce("sum", input, dims, keep_dims)
def reduce_max(input, *dims, keep_dims=False): return _reduce("max", input, dims, keep_dims)
def reduce_min(input, *dims, keep_dims=False): return _reduce("min", input, dims, keep_dims)
def reduce_prod(input, *dims, keep_dims=False): return _reduce("prod", input, dims, keep_dims)


# ------------------------------------------------------------------------------------------------
# creation
# ------------------------------------------------------------------------------------------------
def full(shape, value, dtype: Optional[DataType] = None, location: TileLocation = TileLocation.UB) -> Tile:
    shape = verify_shape(shape)
    v = _scalar(value)
    if dtype is None:
        dtype = v.dtype
    return Tile(shape, dtype, trace.current().node("full", value=v), location)


def full_like(input: Tile, value, location: TileLocation = TileLocation.UB) -> Tile:
    return full(input.shape, value, input.dtype, location)


def zeros(shape, dtype: DataType = KT.int32, location: TileLocation = TileLocation.UB) -> Tile:
    return full(shape, 0, dtype, location)


def zeros_like(input: Tile, location: TileLocation = TileLocation.UB) -> Tile:
    return full(input.shape, 0, input.dtype, location)


def zeros_acc(shape, dtype: DataType) -> Tile:
    shape = verify_shape(shape)
    if len(shape) != 2:
        raise RuntimeError("Accumulator tile must have two dims")
    return Tile(shape, dtype, trace.current().node("zeros_acc"), TileLocation.L0C)


def concat(*inputs: Tile) -> Tile:
    if not inputs or not all(isinstance(t, Tile) for t in inputs):
        raise RuntimeError("All input arguments must be tiles")
    first = inputs[0]
    if any(t.shape[1:] != first.shape[1:] for t in inputs):
        raise RuntimeError("All tiles must have the same shape except their first dimension")
    if any(t.dtype != first.dtype for t in inputs):
        raise RuntimeError("All tiles must have the same dtype")
    shape = (sum(t.shape[0] for t in inputs), ) + first.shape[1:]
    return Tile(shape, first.dtype, trace.current().node("concat", *inputs))


# ------------------------------------------------------------------------------------------------
# shape
# ------------------------------------------------------------------------------------------------
def _flat_shape(shape) -> Tuple[int, ...]:
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    return verify_shape(shape)


def broadcast_to(input: Tile, *shape) -> Tile:
    shape = _flat_shape(shape)
    src = (1, ) * (len(shape) - len(input.shape)) + input.shape
    if len(src) != len(shape) or any(s != d and s != 1 for s, d in zip(src, shape)):
        raise RuntimeError(f"Cannot broadcast {input.shape} to {shape}")
    return Tile(shape, input.dtype, trace.current().node("broadcast", input, shape=shape))


def reshape(input: Tile, *shape) -> Tile:
    shape = _flat_shape(shape)
    n = 1
    for d in shape:
        n *= d
    if n != input.size:
        raise RuntimeError(f"Cannot reshape {input.shape} to {shape}")
    return Tile(shape, input.dtype, trace.current().node("reshape", input, shape=shape))


def ravel(input: Tile) -> Tile:
    return reshape(input, input.size)


def expand_dims(input: Tile, *axis: int) -> Tile:
    shape = list(input.shape)
    for a in sorted(a + len(shape) + 1 if a < 0 else a for a in axis):
        shape.insert(a, 1)
    return reshape(input, *shape)


def squeeze(input: Tile, *axis: int) -> Tile:
    rank = len(input.shape)
    drop = {a + rank if a < 0 else a for a in axis} if axis else {i for i, s in enumerate(input.shape) if s == 1}
    if any(input.shape[a] != 1 for a in drop):
        raise RuntimeError("Only dims of size 1 can be squeezed")
    shape = [s for i, s in enumerate(input.shape) if i not in drop] or [1]
    return reshape(input, *shape)


# ------------------------------------------------------------------------------------------------
# indexing / atomics / programming model
# ------------------------------------------------------------------------------------------------
def where(mask: Tile, src0: Any, src1: Any) -> Tile:
    if not isinstance(mask, Tile):
        raise RuntimeError("'mask' must be a tile")
    dtype = infer_dtype(src0, src1)
    a = src0 if isinstance(src0, Tile) else _scalar(src0)
    b = src1 if isinstance(src1, Tile) else _scalar(src1)
    return Tile(mask.shape, dtype, trace.current().node("where", mask, a, b))


@contextlib.contextmanager
def mask(*, count=None, bits=None, other=None):
    """``with asc2.mask(count=n, other=v):`` -- the unary and binary tile operations inside compute only the first
    ``n`` elements of their tile (row-major order); the remaining elements of each result hold ``v``
    (python/asc/language/tile/indexing_ops.py:30-63; the reference's lowering fills the destination with ``other`` and
    runs the vector instruction under a count mask, lib/Conversion/LowerToAsc/ExpandMask.cpp:36-67).  Without
    ``other`` the reference leaves those elements undefined; here they hold the unmasked result.  The ``bits`` form
    (a raw 128-bit lane mask of the Ascend vector unit) has no counterpart on this platform."""
    if count is None and bits is None:
        raise ValueError("One of 'count', 'bits' must be provided")
    if count is None:
        raise NotImplementedError("asc2.mask(bits=...) addresses the lanes of the Ascend vector unit and is not "
                                  "supported by the CUDA platform; use count=")
    ctx = trace.current()
    entry = (_scalar(count), None if other is None else _scalar(other))
    ctx.masks.append(entry)
    try:
        yield
    finally:
        ctx.masks.pop()


def _masked(result: Tile) -> Tile:
    """Applies the innermost active ``asc2.mask`` to the result of a unary or binary operation."""
    ctx = trace.current()
    if not ctx.masks:
        return result
    count, other = ctx.masks[-1]
    if other is None:
        return result
    index = Tile(result.shape, KT.int32, ctx.node("iota"), result.location)
    active = Tile(result.shape, KT.bool_, ctx.node("compare", index, count, mode="lt"))
    return Tile(result.shape, result.dtype, ctx.node("where", active, result, other), result.location)


def causal_mask(scores: Tile, q_offset: Any, kv_offset: Any) -> Tile:
    """CUDA platform extension: ``scores[i, j] = -inf`` where ``kv_offset + j > q_offset + i``
    (the reference has no index-generating op from which such a mask could be built)."""
    if not isinstance(scores, Tile) or len(scores.shape) != 2 or not scores.dtype.is_float():
        raise RuntimeError("'causal_mask' expects a 2-D floating-point tile")
    node = trace.current().node("causal_mask", scores, q_offset=_scalar(q_offset), kv_offset=_scalar(kv_offset))
    return Tile(scores.shape, scores.dtype, node, scores.location)


def _atomic(kind: str, tile: Tile, tensor: Tensor, offsets: Iterable) -> None:
    trace.current().effect("atomic", tile, tensor, kind=kind, offsets=_offsets(offsets))


def atomic_add(tile, tensor, offsets): _atomic("add", tile, tensor, offsets)
def atomic_max(tile, tensor, offsets): _atomic("max", tile, tensor, offsets)
def atomic_min(tile, tensor, offsets): _atomic("min", tile, tensor, offsets)


def block_idx() -> PlainValue:
    return trace.current().block_idx


def block_num() -> PlainValue:
    return PlainValue.const(trace.current().core_num)


def num_tiles(tensor: Tensor, axis: int, shape: Iterable[int]):
    shape = tuple(shape)
    return (tensor.shape[axis] + shape[axis] - 1) // shape[axis]
