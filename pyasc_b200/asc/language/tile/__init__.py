"""The asc2 tile language (reference: python/asc/language/tile/)."""
from .tensor import Tensor, tensor  # noqa: F401
from .tile import Tile, TileLocation  # noqa: F401
from .range import range, static_range  # noqa: F401
from . import ops  # noqa: F401
