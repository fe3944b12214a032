"""Values a kernel body sees while it is traced.

``GlobalAddress`` stands for a pointer argument and ``PlainValue`` for a scalar
(reference: python/asc/language/core/ir_value.py:36,62).  The reference builds MLIR values; here a
``PlainValue`` is a small symbolic expression over integer/float constants, ``block_idx`` and loop
variables that can be evaluated for all blocks and iterations at once with NumPy, which is how the
launcher works out which part of each tensor a kernel touches.

Scalar semantics follow the reference (ir_value.py:76-97): ``+ - *`` as usual, both ``/`` and
``//`` are truncating signed division on integers, ``%`` is the signed remainder.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple, Union

import numpy as np

from .dtype import DataType, KnownTypes as KT

Number = Union[int, float, bool]


class GlobalAddress:
    """Pointer to global (device) memory.  Used as an annotation in kernel signatures and, during
    tracing, as the value bound to the pointer parameter."""

    def __init__(self, name: str = "", dtype: Optional[DataType] = None, index: int = -1, numel: int = 0):
        self.name = name
        self.dtype = dtype
        self.index = index    # position among the runtime arguments
        self.numel = numel    # elements in the caller's buffer

    def __repr__(self) -> str:
        return f"GlobalAddress({self.name}: {self.dtype}*)"


_INT_OPS = {"add", "sub", "mul", "div", "mod", "min", "max", "neg"}
_CMP_OPS = {"lt", "le", "gt", "ge", "eq", "ne"}


def _trunc_div(a, b):
    a = np.asarray(a)
    b = np.asarray(b)
    if np.issubdtype(a.dtype, np.integer) and np.issubdtype(b.dtype, np.integer):
        q = np.abs(a) // np.abs(b)
        return np.where((a < 0) != (b < 0), -q, q)
    return a / b


def _apply(op: str, vals):
    if op == "add":
        return vals[0] + vals[1]
    if op == "sub":
        return vals[0] - vals[1]
    if op == "mul":
        return vals[0] * vals[1]
    if op == "div":
        return _trunc_div(vals[0], vals[1])
    if op == "mod":
        return np.fmod(vals[0], vals[1])
    if op == "min":
        return np.minimum(vals[0], vals[1])
    if op == "max":
        return np.maximum(vals[0], vals[1])
    if op == "neg":
        return -vals[0]
    if op == "lt":
        return vals[0] < vals[1]
    if op == "le":
        return vals[0] <= vals[1]
    if op == "gt":
        return vals[0] > vals[1]
    if op == "ge":
        return vals[0] >= vals[1]
    if op == "eq":
        return vals[0] == vals[1]
    if op == "ne":
        return vals[0] != vals[1]
    raise NotImplementedError(op)


class PlainValue:
    """A traced scalar: constant, symbol, or an arithmetic expression over those."""

    __slots__ = ("op", "args", "dtype")

    def __init__(self, op: str, args: Tuple[Any, ...], dtype: DataType):
        self.op = op
        self.args = args
        self.dtype = dtype

    # ---- construction -------------------------------------------------------------------------
    @staticmethod
    def const(value: Number, dtype: Optional[DataType] = None) -> "PlainValue":
        if dtype is None:
            dtype = KT.bool_ if isinstance(value, bool) else KT.int32 if isinstance(value, (int, np.integer)) \
                else KT.float32
        return PlainValue("const", (value, ), dtype)

    @staticmethod
    def sym(name: str, dtype: DataType = KT.int32) -> "PlainValue":
        return PlainValue("sym", (name, ), dtype)

    @staticmethod
    def wrap(value: Any) -> "PlainValue":
        if isinstance(value, PlainValue):
            return value
        if isinstance(value, (bool, int, float, np.integer, np.floating)):
            return PlainValue.const(value.item() if isinstance(value, np.generic) else value)
        raise TypeError(f"Cannot use {type(value).__name__} as a scalar value")

    # ---- queries ------------------------------------------------------------------------------
    @property
    def is_const(self) -> bool:
        return self.op == "const"

    @property
    def value(self) -> Number:
        if not self.is_const:
            raise RuntimeError("Scalar is not a compile-time constant")
        return self.args[0]

    def symbols(self) -> set:
        if self.op == "sym":
            return {self.args[0]}
        out = set()
        for a in self.args:
            if isinstance(a, PlainValue):
                out |= a.symbols()
        return out

    def evaluate(self, env: Dict[str, Any]):
        """Value for the symbol bindings in ``env`` (scalars or broadcastable NumPy arrays)."""
        if self.op == "const":
            return self.args[0]
        if self.op == "sym":
            return env[self.args[0]]
        if self.op == "tile_scalar":
            raise NotImplementedError("A scalar computed from tile data has no launch-time value")
        return _apply(self.op, [a.evaluate(env) for a in self.args])

    # ---- arithmetic ---------------------------------------------------------------------------
    def _bin(self, op: str, other: Any, reverse: bool = False) -> "PlainValue":
        try:
            other = PlainValue.wrap(other)
        except TypeError:
            return NotImplemented
        lhs, rhs = (other, self) if reverse else (self, other)
        if op in _CMP_OPS:
            dtype = KT.bool_
        elif lhs.dtype.is_float() or rhs.dtype.is_float():
            dtype = lhs.dtype if lhs.dtype.is_float() else rhs.dtype
        else:
            dtype = lhs.dtype if lhs.dtype.bitwidth >= rhs.dtype.bitwidth else rhs.dtype
        if lhs.is_const and rhs.is_const:
            a, b = lhs.value, rhs.value
            if op in ("div", "mod") and not dtype.is_float() and b == 0:
                raise ZeroDivisionError("division by zero in a kernel scalar expression")
            res = _apply(op, [a, b])
            res = res.item() if isinstance(res, (np.generic, np.ndarray)) else res
            return PlainValue.const(res, dtype)
        return PlainValue(op, (lhs, rhs), dtype)

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __truediv__(self, o): return self._bin("div", o)
    def __rtruediv__(self, o): return self._bin("div", o, True)
    def __floordiv__(self, o): return self._bin("div", o)
    def __rfloordiv__(self, o): return self._bin("div", o, True)
    def __mod__(self, o): return self._bin("mod", o)
    def __rmod__(self, o): return self._bin("mod", o, True)
    def __lt__(self, o): return self._bin("lt", o)
    def __le__(self, o): return self._bin("le", o)
    def __gt__(self, o): return self._bin("gt", o)
    def __ge__(self, o): return self._bin("ge", o)
    def __eq__(self, o): return self._bin("eq", o)  # type: ignore[override]
    def __ne__(self, o): return self._bin("ne", o)  # type: ignore[override]
    __hash__ = None  # type: ignore[assignment]

    def __neg__(self):
        if self.is_const:
            return PlainValue.const(-self.value, self.dtype)
        return PlainValue("neg", (self, ), self.dtype)

    def __pos__(self):
        return self

    def ceildiv(self, other):
        return (self + other - 1) // other

    def __bool__(self) -> bool:
        if self.is_const:
            return bool(self.value)
        # a condition on the block index or a loop variable: the tracer follows one outcome per run and records it
        # (the reference emits scf.if, python/asc/codegen/function_visitor.py:585-627)
        from ..tile import trace
        if trace.is_tracing():
            return trace.current().branch(self)
        raise NotImplementedError("Branching on a run-time scalar outside a kernel")

    def __index__(self) -> int:
        if self.is_const and not self.dtype.is_float():
            return int(self.value)
        raise TypeError("A run-time scalar cannot be used where a Python integer is required")

    def __int__(self) -> int:
        return int(self.value)

    def __float__(self) -> float:
        return float(self.value)

    def __repr__(self) -> str:
        if self.op == "const":
            return f"{self.args[0]!r}"
        if self.op == "sym":
            return f"%{self.args[0]}"
        return f"{self.op}({', '.join(map(repr, self.args))})"

    def key(self) -> tuple:
        """Hashable structural identity (PlainValue itself is unhashable because == is symbolic)."""
        if self.op in ("const", "sym"):
            return (self.op, self.args[0])
        return (self.op, ) + tuple(a.key() if isinstance(a, PlainValue) else ("node", getattr(a, "uid", id(a)))
                                   for a in self.args)


def same_scalar(a: Any, b: Any) -> bool:
    """Structural equality of two scalars (PlainValue or Python numbers)."""
    return PlainValue.wrap(a).key() == PlainValue.wrap(b).key()


RuntimeInt = Union[int, PlainValue]
RuntimeFloat = Union[float, PlainValue]
RuntimeNumeric = Union[int, float, bool, PlainValue]
