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


class _Signatures:
    """Structural digests of traced values: two values recorded by different runs of the kernel get the same digest
    when they are the same computation (same operations on the same tensors at the same offsets inside loops with the
    same bounds).  Digests are computed bottom-up and memoised per object, so shared subexpressions cost once."""

    def __init__(self):
        self._memo: Dict[int, str] = {}
        self._keep: List[Any] = []        # the memo is keyed by id(): keep the objects alive

    def of(self, x: Any) -> str:
        from ..language.tile.tensor import Tensor
        from ..language.tile.tile import Tile
        from ..language.tile.trace import Loop, Node
        if isinstance(x, (Tile, Node, PlainValue, Tensor, Loop, Effect)):
            key = id(x)
            hit = self._memo.get(key)
            if hit is not None:
                return hit
            if isinstance(x, Tile):
                parts = ("T", repr(x.shape), x.dtype.name, self.of(x.node))
            elif isinstance(x, Node):
                parts = ("N", x.kind, self.of(x.args), self.of(x.attrs), self.of(x.loops))
            elif isinstance(x, PlainValue):
                parts = ("P", x.op, x.dtype.name, self.of(x.args))
            elif isinstance(x, Tensor):
                parts = ("X", repr(x.base.index), x.dtype.name, self.of(x.shape))
            elif isinstance(x, Loop):
                parts = ("L", x.name, self.of(x.start), self.of(x.stop), self.of(x.step))
            else:
                parts = ("E", x.kind, self.of(x.args), self.of(x.attrs), self.of(x.loops))
            import hashlib
            digest = hashlib.blake2b("\x1f".join(parts).encode(), digest_size=12).hexdigest()
            self._memo[key] = digest
            self._keep.append(x)
            return digest
        if isinstance(x, (tuple, list)):
            return "(" + ",".join(self.of(v) for v in x) + ")"
        if isinstance(x, dict):
            return "{" + ",".join(f"{k}:{self.of(v)}" for k, v in sorted(x.items(), key=lambda kv: str(kv[0]))) + "}"
        if isinstance(x, GlobalAddress):
            return f"G{x.index!r}"
        return repr(x)


def _merge_paths(effects: List[Effect]) -> List[Effect]:
    """Statements after an ``if`` on a run-time scalar are traced once per path, so each shows up as several effects
    that differ only in the outcome of that ``if``.  Two effects that are the same computation under guards that agree
    except for opposite outcomes of one condition happen whichever way that condition goes: they become one effect
    without it (repeatedly, for nests and sequences of ``if``s).  The merged effect takes the place of the
    earlier one; the two never both happen for one block and iteration."""
    if not any(e.guards for e in effects):
        return effects
    sig = _Signatures()
    effects = list(effects)
    merged = True
    while merged:
        merged = False
        seen: Dict[tuple, int] = {}
        for i, e in enumerate(effects):
            if not e.guards:
                continue
            body = sig.of(e)
            conds = [sig.of(c) for c, _ in e.guards]
            hit = None
            for k, (_, outcome) in enumerate(e.guards):
                # the same computation under the same guards except for the other outcome of condition k
                others = tuple((c, o) for j, ((_, o), c) in enumerate(zip(e.guards, conds)) if j != k)
                key = (body, k, conds[k], others)
                j = seen.get(key + (not outcome, ))
                if j is not None:
                    hit = (j, k)
                    break
                seen[key + (outcome, )] = i
            if hit is not None:
                j, k = hit
                effects[j].guards = effects[j].guards[:k] + effects[j].guards[k + 1:]
                del effects[i]
                merged = True
                break
    return effects


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
    return KernelTrace(fn.__name__, core_num, _merge_paths(effects), pointers)
