"""asc2 atomic ops (same module path as the reference: python/asc/language/tile/atomic_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    atomic_add,
    atomic_max,
    atomic_min,
)

__all__ = ["atomic_add", "atomic_max", "atomic_min"]
