"""asc2 creation ops (same module path as the reference: python/asc/language/tile/creation_ops.py);
the implementations live in :mod:`asc.language.tile.ops`."""
from .ops import (  # noqa: F401
    concat,
    full,
    full_like,
    zeros,
    zeros_acc,
    zeros_like,
)

__all__ = ["concat", "full", "full_like", "zeros", "zeros_acc", "zeros_like"]
