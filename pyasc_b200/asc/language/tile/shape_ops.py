"""asc2 shape ops (same module path as the reference: python/asc/language/tile/shape_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    broadcast_to,
    expand_dims,
    ravel,
    reshape,
    squeeze,
)

__all__ = ["broadcast_to", "expand_dims", "ravel", "reshape", "squeeze"]
