"""Shape / dtype inference shared by the tile ops
(reference: python/asc/language/tile/utils.py:49-139)."""
from __future__ import annotations

from typing import Any, Iterable, Tuple

from ..core.dtype import DataType, KnownTypes as KT
from ..core.ir_value import PlainValue
from .tile import Tile

UB_BLOCK_SIZE = 32  # bytes; the reference's alignment unit for the last tile dimension (python/src/IR.cpp:99)


def verify_shape(shape: Iterable[int], name: str = "shape") -> Tuple[int, ...]:
    shape = tuple(int(d) if isinstance(d, PlainValue) and d.is_const else d for d in shape)
    if len(shape) < 1:
        raise RuntimeError(f"'{name}' must have at least one value")
    if not all(isinstance(dim, int) and not isinstance(dim, bool) for dim in shape):
        raise RuntimeError(f"All values in '{name}' must be integers")
    if any(dim <= 0 for dim in shape):
        raise RuntimeError(f"All values in '{name}' must be positive")
    return shape


def check_data_alignment(shape: Tuple[int, ...], dtype: DataType) -> None:
    try:
        dtype_size = dtype.sizeof()
    except ValueError:
        return
    if len(shape) > 1 and shape[-1] % (UB_BLOCK_SIZE // dtype_size) != 0:
        raise RuntimeError(f"Last dimension of tile must be aligned by {UB_BLOCK_SIZE} bytes, "
                           f"got {shape[-1]} x {dtype_size} bytes")


def _scalar_dtype(v: Any) -> DataType:
    if isinstance(v, (Tile, PlainValue)):
        return v.dtype
    if isinstance(v, bool):
        return KT.bool_
    if isinstance(v, int):
        return KT.int32
    if isinstance(v, float):
        return KT.float32
    raise RuntimeError(f"Cannot infer a dtype for {type(v).__name__}")


def infer_dtype(lhs: Any, rhs: Any) -> DataType:
    """Common dtype of two operands: a tile's dtype wins over a scalar's; between two tiles or two
    scalars of one kind the wider wins, and float wins over int of the same width
    (reference: python/asc/language/tile/utils.py:73-94)."""
    a, b = _scalar_dtype(lhs), _scalar_dtype(rhs)
    if a == b:
        return a
    if a.is_unsigned() or b.is_unsigned():
        raise NotImplementedError(f"Unsigned dtype operands not supported, got {a} and {b}")
    lt, rt = isinstance(lhs, Tile), isinstance(rhs, Tile)
    if lt and not rt:
        return a
    if rt and not lt:
        return b
    if a.is_float() == b.is_float() and a.bitwidth != b.bitwidth:
        return a if a.bitwidth > b.bitwidth else b
    if a.bitwidth == b.bitwidth:
        return a if a.is_float() else b
    if lt and rt:
        return a if a.is_float() else b   # mixed kinds and widths between tiles: the float one
    raise RuntimeError(f"Unable to infer common dtype between {a} and {b}")


def infer_shape(lhs: Any, rhs: Any) -> Tuple[int, ...]:
    lt, rt = isinstance(lhs, Tile), isinstance(rhs, Tile)
    if lt and rt:
        if lhs.shape == rhs.shape:
            return lhs.shape
        raise RuntimeError(f"Shape mismatch: {lhs.shape} vs. {rhs.shape}")
    return lhs.shape if lt else rhs.shape


def default_float() -> DataType:
    return KT.float32
