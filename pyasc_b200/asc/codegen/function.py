"""Kernel function wrapper: source identity and the runtime / compile-time argument split
(reference: python/asc/codegen/function.py:63-132)."""
from __future__ import annotations

import hashlib
import inspect
from typing import Any, Callable, Dict, Generic, Tuple, TypeVar, get_args, get_origin

from typing_extensions import ParamSpec

from ..language.core.constexpr import ConstExpr, require_constexpr

P = ParamSpec("P")
T = TypeVar("T")


def get_annotations(fn: Callable) -> Dict[str, Any]:
    try:
        return inspect.get_annotations(fn, eval_str=True)
    except Exception:
        return dict(getattr(fn, "__annotations__", {}))


class Function(Generic[P, T]):

    def __init__(self, fn: Callable[P, T]):
        self.fn = fn
        self.fn_name = fn.__name__
        try:
            self.src = inspect.getsource(fn)
        except (OSError, TypeError):
            self.src = fn.__code__.co_code.hex()
        self.__name__ = fn.__name__
        self.__doc__ = fn.__doc__

    @property
    def cache_key(self) -> str:
        return hashlib.blake2b(self.src.encode("utf-8"), digest_size=16).hexdigest()

    @staticmethod
    def split_args(args: Dict[str, Any], annotations: Dict[str, Any]) -> Tuple[Dict[str, Any], Dict[str, ConstExpr]]:
        """``asc.ConstExpr[...]``-annotated parameters are compile-time values, the rest run-time."""
        runtime_args: Dict[str, Any] = {}
        constexprs: Dict[str, ConstExpr] = {}
        for name, value in args.items():
            ann_type = annotations.get(name, object)
            origin = get_origin(ann_type) or ann_type
            if isinstance(origin, type) and issubclass(origin, ConstExpr):
                ann_args = get_args(ann_type)
                if len(ann_args) != 0:
                    require_constexpr(value, *ann_args, arg_name=name)
                constexprs[name] = ConstExpr(value)
            else:
                runtime_args[name] = value
        return runtime_args, constexprs

    def __call__(self, *args: P.args, **kwargs: P.kwargs) -> T:
        raise RuntimeError("Kernel must be launched as kernel[core_num](...)")
