"""``Tile``: a statically shaped on-chip array value
(reference: python/asc/language/tile/tile.py:24-290)."""
from __future__ import annotations

from enum import Enum
from typing import Tuple

from ..core.dtype import DataType
from .trace import Node


class TileLocation(Enum):
    """Where the reference places a tile on the Ascend core (python/src/IR.cpp:206-212).  On the
    CUDA platform the location only tells the matcher which role a tile plays (vector operand,
    matmul A/B operand, staged copy)."""
    UB = "UB"
    L1 = "L1"
    L0A = "L0A"
    L0B = "L0B"
    L0C = "L0C"


class BinaryOperandTypeError(TypeError):
    pass


class Tile:

    def __init__(self, shape: Tuple[int, ...], dtype: DataType, node: Node, location: TileLocation = TileLocation.UB):
        self.shape = tuple(shape)
        self.dtype = dtype
        self.node = node
        self.location = location

    @property
    def size(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def __repr__(self) -> str:
        return f"Tile({list(self.shape)} x {self.dtype}, {self.location.value}, {self.node.kind}#{self.node.uid})"

    def __bool__(self) -> bool:
        raise NotImplementedError("A tile has no truth value; use asc2.where")

    __hash__ = object.__hash__

    def to(self, dtype: DataType) -> "Tile":
        from . import ops
        return ops.cast(self, dtype)

    # binary
    def __add__(self, o): from . import ops; return ops.add(self, o)
    def __radd__(self, o): from . import ops; return ops.add(o, self)
    def __sub__(self, o): from . import ops; return ops.sub(self, o)
    def __rsub__(self, o): from . import ops; return ops.sub(o, self)
    def __mul__(self, o): from . import ops; return ops.mul(self, o)
    def __rmul__(self, o): from . import ops; return ops.mul(o, self)
    def __truediv__(self, o): from . import ops; return ops.div(self, o)
    def __rtruediv__(self, o): from . import ops; return ops.div(o, self)
    def __floordiv__(self, o): from . import ops; return ops.div(self, o)
    def __lshift__(self, o): from . import ops; return ops.left_shift(self, o)
    def __rshift__(self, o): from . import ops; return ops.right_shift(self, o)
    def __matmul__(self, o): from . import ops; return ops.matmul(self, o)
    def __eq__(self, o): from . import ops; return ops.equal(self, o)  # type: ignore[override]
    def __ne__(self, o): from . import ops; return ops.not_equal(self, o)  # type: ignore[override]
    def __gt__(self, o): from . import ops; return ops.greater(self, o)
    def __ge__(self, o): from . import ops; return ops.greater_equal(self, o)
    def __lt__(self, o): from . import ops; return ops.less(self, o)
    def __le__(self, o): from . import ops; return ops.less_equal(self, o)
    def __neg__(self): from . import ops; return ops.negative(self)
    def __pos__(self): return self

    # reductions
    def sum(self, *dims, keep_dims=False): from . import ops; return ops.reduce_sum(self, *dims, keep_dims=keep_dims)
    def max(self, *dims, keep_dims=False): from . import ops; return ops.reduce_max(self, *dims, keep_dims=keep_dims)
    def min(self, *dims, keep_dims=False): from . import ops; return ops.reduce_min(self, *dims, keep_dims=keep_dims)
    def prod(self, *dims, keep_dims=False): from . import ops; return ops.reduce_prod(self, *dims, keep_dims=keep_dims)

    # shape
    def broadcast_to(self, *shape): from . import ops; return ops.broadcast_to(self, *shape)
    def reshape(self, *shape): from . import ops; return ops.reshape(self, *shape)
    def ravel(self): from . import ops; return ops.ravel(self)
    def expand_dims(self, *axis): from . import ops; return ops.expand_dims(self, *axis)
    def squeeze(self, *axis): from . import ops; return ops.squeeze(self, *axis)


def _bind_unary(name: str) -> None:
    def method(self):
        from . import ops
        return getattr(ops, name)(self)
    method.__name__ = name
    setattr(Tile, name, method)


for _n in ("sin", "cos", "tan", "sinh", "cosh", "tanh", "exp", "log", "log2", "floor", "ceil", "abs", "erf", "exp2",
           "sqrt", "rsqrt", "relu"):
    _bind_unary(_n)
