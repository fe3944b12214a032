"""Names kernels refer to as ``asc.<name>`` (reference: python/asc/language/__init__.py).  Only the
part of the ``asc`` (v1) language that asc2 kernels touch is provided."""
from .core.constexpr import ConstExpr, require_constexpr
from .core.dtype import (DataType, KnownTypes, bfloat16, bool_, float16, float32, float64, half, int8, int16,
                         int32, int64, uint8, uint16, uint32, uint64)
from .core.ir_value import GlobalAddress, PlainValue
from .core.utils import ceildiv, number
from .tile.range import static_range
from .tile.ops import block_idx as get_block_idx, block_num as get_block_num

__all__ = [
    "ConstExpr", "require_constexpr", "DataType", "KnownTypes", "bfloat16", "bool_", "float16", "float32", "float64",
    "half", "int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64", "GlobalAddress", "PlainValue",
    "ceildiv", "number", "static_range", "get_block_idx", "get_block_num",
]
