"""Small host-side helpers (reference: python/asc/language/core/utils.py:173)."""


def ceildiv(a, b):
    """Ceiling division for ints and traced scalars alike."""
    return -(-a // b) if isinstance(a, int) and isinstance(b, int) else (a + b - 1) // b
