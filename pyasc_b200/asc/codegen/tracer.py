"""Runs a kernel function once with proxy arguments and returns what it recorded.

Stands in for the reference's AST walk (python/asc/codegen/function_visitor.py:560-583): pointer
arguments become ``GlobalAddress`` proxies, run-time scalars become ``PlainValue`` constants holding
the value of this launch (int -> int32, float -> float32, as in
python/asc/runtime/launcher.py:142-145; 0-dim tensors keep their dtype), ConstExpr arguments are
plain Python values, and ``range`` inside the kernel body resolves to the custom builtin given by the
decorator (``asc2.range``), as in python/asc/codegen/name_scope.py:15-35.
"""
from __future__ import annotations

import types
from typing import Any, Callable, Dict, List, Optional

import numpy as np

from ..language.core.constexpr import ConstExpr
from ..language.core.dtype import DataType, KnownTypes as KT
from ..language.core.ir_value import GlobalAddress, PlainValue
from ..language.tile.trace import Effect, TraceContext


class CodegenError(RuntimeError):
    pass


class KernelTrace:
    """Everything one traced launch recorded."""

    def __init__(self, fn_name: str, core_num: int, effects: List[Effect], pointers: List[GlobalAddress]):
        self.fn_name = fn_name
        self.core_num = core_num
        self.effects = effects
        self.pointers = pointers


def _scalar_proxy(value: Any) -> Optional[PlainValue]:
    if isinstance(value, bool):
        return PlainValue.const(int(value), KT.int32)
    if isinstance(value, int):
        return PlainValue.const(value, KT.int32)
    if isinstance(value, float):
        return PlainValue.const(float(np.float32(value)), KT.float32)
    if isinstance(value, np.generic):
        return PlainValue.const(value.item(), DataType(str(value.dtype)))
    try:
        import torch
        if isinstance(value, torch.Tensor) and value.dim() == 0:
            return PlainValue.const(value.item(), DataType(str(value.dtype)))
    except ModuleNotFoundError:
        pass
    return None


def _pointer_proxy(name: str, value: Any, index: int) -> Optional[GlobalAddress]:
    if isinstance(value, np.ndarray):
        return GlobalAddress(name, DataType(str(value.dtype)), index, int(value.size))
    try:
        import torch
        if isinstance(value, torch.Tensor) and value.dim() > 0:
            return GlobalAddress(name, DataType(str(value.dtype)), index, int(value.numel()))
    except ModuleNotFoundError:
        pass
    return None


MAX_PATHS = 64      # paths through ``if``s on run-time scalars one kernel may have


def trace_kernel(fn: Callable, runtime_args: Dict[str, Any], constexprs: Dict[str, ConstExpr], core_num: int,
                 custom_builtins: Optional[Dict[str, Any]] = None, unroll_limit: int = 0) -> KernelTrace:
    call_args: Dict[str, Any] = {}
    pointers: List[GlobalAddress] = []
    for index, (name, value) in enumerate(runtime_args.items()):
        scalar = _scalar_proxy(value)
        if scalar is not None:
            call_args[name] = scalar
            continue
        ptr = _pointer_proxy(name, value, index)
        if ptr is None:
            raise TypeError(f"Argument type in JIT function is not supported: {value.__class__.__name__}")
        pointers.append(ptr)
        call_args[name] = ptr
    for name, value in constexprs.items():
        call_args[name] = ConstExpr.unwrap(value)

    scope = dict(fn.__globals__)
    scope.update(custom_builtins or {})
    traced_fn = types.FunctionType(fn.__code__, scope, fn.__name__, fn.__defaults__, fn.__closure__)
    traced_fn.__kwdefaults__ = fn.__kwdefaults__

    # One run per path through the kernel's ``if``s on run-time scalars (depth first).  A run that was forced down
    # its first m branches shares everything before the m-th branch with the run it was forked from, so only the
    # effects it recorded after that branch are new.
    effects: List[Effect] = []
    pending: List[tuple] = [()]
    runs = 0
    while pending:
        forced = pending.pop()
        runs += 1
        if runs > MAX_PATHS:
            raise NotImplementedError(f"kernel '{fn.__name__}' branches on run-time scalars along more than {MAX_PATHS} paths")
        with TraceContext(fn.__name__, core_num, forced, unroll_limit) as ctx:
            traced_fn(**call_args)
            if ctx.loops:
                raise CodegenError("Unbalanced loop nest at the end of kernel tracing")
        effects += [e for e in ctx.effects if len(e.guards) >= len(forced)]
        outcomes = tuple(o for _, o in ctx.taken)
        for j in range(len(ctx.taken) - 1, len(forced) - 1, -1):
            pending.append(outcomes[:j] + (not outcomes[j], ))
    return KernelTrace(fn.__name__, core_num, effects, pointers)
