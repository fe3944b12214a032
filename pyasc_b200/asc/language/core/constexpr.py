"""Compile-time arguments (reference: python/asc/language/core/constexpr.py:21-72).

A kernel parameter annotated ``asc.ConstExpr[...]`` is a plain Python value while the kernel body
is traced; everything else is a runtime argument.
"""
from __future__ import annotations

from typing import Any, Generic, Optional, Type, TypeVar, Union

T_co = TypeVar("T_co", covariant=True)


class ConstExpr(Generic[T_co]):
    value: T_co

    def __init__(self, value):
        self.value = self.unwrap(value)

    def __str__(self) -> str:
        return str(self.value)

    def __repr__(self) -> str:
        return f"ConstExpr[{self.value.__class__.__name__}]({self.value!r})"

    def __format__(self, format_spec: str) -> str:
        return ("{:%s}" % (format_spec, )).format(self.value)

    @staticmethod
    def unwrap(obj):
        return obj.value if isinstance(obj, ConstExpr) else obj


def require_constexpr(obj: Union[ConstExpr, Any], *constraints: Type, arg_name: Optional[str] = None) -> None:
    """Raise unless ``obj`` (or the value it wraps) is an instance of one of ``constraints``."""
    if len(constraints) == 0:
        raise RuntimeError("Constraints must be provided for ConstExpr requirement")
    value = ConstExpr.unwrap(obj)
    real = tuple(c for c in constraints if isinstance(c, type))
    if not real or isinstance(value, real):
        return
    names = " | ".join(getattr(c, "__name__", str(c)) for c in constraints)
    note = "" if arg_name is None else f" for '{arg_name}' argument"
    raise RuntimeError(f"ConstExpr[{names}] is required{note}, {value.__class__.__name__} was provided: {value}")
