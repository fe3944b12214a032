"""asc2 reduction ops (same module path as the reference: python/asc/language/tile/reduction_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    reduce_max,
    reduce_min,
    reduce_sum,
    reduce_prod,
)

__all__ = ["reduce_max", "reduce_min", "reduce_sum", "reduce_prod"]
