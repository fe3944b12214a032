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


def infer_dtype(lhs: Any, rhs: Any) -> DataType:
    """Tile dtype wins over a scalar; between tiles of one kind the wider wins
    (reference: utils.py:73-94)."""
    lt, rt = isinstance(lhs, Tile), isinstance(rhs, Tile)
    if lt and rt:
        a, b = lhs.dtype, rhs.dtype
        if a == b:
            return a
        if a.is_unsigned() or b.is_unsigned():
            raise RuntimeError(f"Unsigned tile types are not supported in binary operations: {a}, {b}")
        if a.is_float() != b.is_float():
            return a if a.is_float() else b
        return a if a.bitwidth >= b.bitwidth else b
    if lt:
        return lhs.dtype
    if rt:
        return rhs.dtype
    raise RuntimeError("At least one operand must be a tile")


def infer_shape(lhs: Any, rhs: Any) -> Tuple[int, ...]:
    lt, rt = isinstance(lhs, Tile), isinstance(rhs, Tile)
    if lt and rt:
        if lhs.shape == rhs.shape:
            return lhs.shape
        raise RuntimeError(f"Shape mismatch: {lhs.shape} vs. {rhs.shape}")
    return lhs.shape if lt else rhs.shape


def default_float() -> DataType:
    return KT.float32
