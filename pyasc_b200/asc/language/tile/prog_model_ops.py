"""asc2 prog model ops (same module path as the reference: python/asc/language/tile/prog_model_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    block_idx,
    block_num,
    num_tiles,
)

__all__ = ["block_idx", "block_num", "num_tiles"]
