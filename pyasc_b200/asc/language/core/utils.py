"""Small host-side helpers (reference: python/asc/language/core/utils.py:173)."""


def ceildiv(a, b):
    """Ceiling division for ints and traced scalars alike."""
    return -(-a // b) if isinstance(a, int) and isinstance(b, int) else (a + b - 1) // b


def number(value, dtype):
    """A scalar constant of a given type (reference: python/asc/language/core/ops.py:33)."""
    from .ir_value import PlainValue
    if isinstance(value, PlainValue):
        value = value.value
    return PlainValue.const(float(value) if dtype.is_float() else int(value), dtype)
