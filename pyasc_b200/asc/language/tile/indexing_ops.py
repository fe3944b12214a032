"""asc2 indexing ops (same module path as the reference: python/asc/language/tile/indexing_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    mask,
    where,
    causal_mask,
)

__all__ = ["mask", "where", "causal_mask"]
