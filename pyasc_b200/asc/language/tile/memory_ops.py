"""asc2 memory ops (same module path as the reference: python/asc/language/tile/memory_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    copy,
    load,
    store,
)

__all__ = ["copy", "load", "store"]
