"""``asc2.tensor``: a row-major N-D view of a global pointer
(reference: python/asc/language/tile/tensor.py:64-116, TensorOp in Ops.td:36)."""
from __future__ import annotations

from typing import Iterable, Tuple

from ..core.dtype import DataType
from ..core.ir_value import GlobalAddress, PlainValue
from . import trace


class Tensor:
    """Contiguous row-major tensor in global memory.  Dimensions are Python ints or traced scalars
    whose value is known at launch."""

    def __init__(self, base: GlobalAddress, shape: Tuple[PlainValue, ...]):
        self.base = base
        self.shape = shape

    @property
    def dtype(self) -> DataType:
        return self.base.dtype

    @property
    def rank(self) -> int:
        return len(self.shape)

    def static_shape(self) -> Tuple[int, ...]:
        out = []
        for d in self.shape:
            if not d.is_const:
                raise NotImplementedError("Tensor dimensions that depend on block_idx or loop variables are not "
                                          "supported by the CUDA platform")
            out.append(int(d.value))
        return tuple(out)

    def __repr__(self) -> str:
        return f"Tensor({self.base.name}, shape={list(self.shape)}, dtype={self.dtype})"


def tensor(base: GlobalAddress, shape: Iterable) -> Tensor:
    if not isinstance(base, GlobalAddress):
        raise TypeError(f"'base' must be a GlobalAddress kernel argument, got {type(base).__name__}")
    dims = tuple(PlainValue.wrap(d) for d in shape)
    if len(dims) < 1:
        raise RuntimeError("'shape' must have at least one value")
    t = Tensor(base, dims)
    trace.current().tensors.append(t)
    return t
