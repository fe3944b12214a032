"""asc2 unary ops (same module path as the reference: python/asc/language/tile/unary_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    abs,
    ceil,
    cos,
    cosh,
    erf,
    exp,
    exp2,
    floor,
    log,
    log2,
    negative,
    relu,
    rms_norm,
    rsqrt,
    sin,
    sinh,
    softmax,
    sqrt,
    tan,
    tanh,
)

__all__ = ["abs", "ceil", "cos", "cosh", "erf", "exp", "exp2", "floor", "log", "log2", "negative", "relu", "rms_norm", "rsqrt", "sin", "sinh", "softmax", "sqrt", "tan", "tanh"]
