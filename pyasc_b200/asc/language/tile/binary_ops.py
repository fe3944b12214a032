"""asc2 binary ops (same module path as the reference: python/asc/language/tile/binary_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    add,
    div,
    equal,
    greater,
    greater_equal,
    left_shift,
    less,
    less_equal,
    matmul,
    matmul_acc,
    maximum,
    minimum,
    mul,
    not_equal,
    right_shift,
    sub,
)

__all__ = ["add", "div", "equal", "greater", "greater_equal", "left_shift", "less", "less_equal", "matmul", "matmul_acc", "maximum", "minimum", "mul", "not_equal", "right_shift", "sub"]
