"""Recording context of the CUDA platform's kernel tracer.

The reference walks the kernel's AST and emits one ``asctile`` MLIR op per asc2 call
(python/asc/codegen/function_visitor.py:463-583; ops in
include/ascir/Dialect/AscTile/IR/Ops.td:28-394).  Here the kernel function itself is executed once
with proxy arguments: every asc2 call appends a :class:`Node` to the active :class:`TraceContext`,
``asc2.range`` loops run their body once with a symbolic induction variable, and stores /
accumulations are kept as an ordered effect list.  The result carries the same information as the
reference's recorded IR and is what the launcher pattern-matches against the CUDA kernels.
"""
from __future__ import annotations

import itertools
from typing import Any, List, Optional, Tuple

from ..core.ir_value import PlainValue

_current: Optional["TraceContext"] = None


class Loop:
    """One ``for`` over ``asc2.range``: ``var`` takes start, start+step, ... < stop."""

    __slots__ = ("var", "start", "stop", "step", "unroll_factor", "parallel")

    def __init__(self, var: PlainValue, start, stop, step, unroll_factor: int, parallel: bool):
        self.var = var
        self.start = PlainValue.wrap(start)
        self.stop = PlainValue.wrap(stop)
        self.step = PlainValue.wrap(step)
        self.unroll_factor = unroll_factor
        self.parallel = parallel

    @property
    def name(self) -> str:
        return self.var.args[0]

    def __repr__(self) -> str:
        return f"for %{self.name} in range({self.start!r}, {self.stop!r}, {self.step!r})"


class Node:
    """One recorded tile operation."""

    __slots__ = ("kind", "args", "attrs", "loops", "uid")
    _ids = itertools.count()

    def __init__(self, kind: str, args: Tuple[Any, ...] = (), attrs: Optional[dict] = None,
                 loops: Tuple[Loop, ...] = ()):
        self.kind = kind
        self.args = args
        self.attrs = attrs or {}
        self.loops = loops
        self.uid = next(Node._ids)

    def __repr__(self) -> str:
        return f"Node#{self.uid}({self.kind}, attrs={self.attrs})"


class Effect:
    """A side effect in program order: ``store``, ``matmul_acc`` or ``atomic``."""

    __slots__ = ("kind", "args", "attrs", "loops", "uid", "guards")

    def __init__(self, kind: str, args: Tuple[Any, ...], attrs: dict, loops: Tuple[Loop, ...],
                 guards: Tuple[Tuple[PlainValue, bool], ...] = ()):
        self.kind = kind
        self.args = args
        self.attrs = attrs
        self.loops = loops
        self.uid = next(Node._ids)    # one counter with the nodes: program order of operations and effects
        # (condition, outcome) of every ``if`` on a run-time scalar this effect lies under: it happens only for the
        # blocks and iterations in which each condition has that outcome
        self.guards = guards

    def __repr__(self) -> str:
        return f"Effect({self.kind}, {self.attrs}, loops={list(self.loops)})"


class TraceContext:

    def __init__(self, fn_name: str, core_num: int, forced: Tuple[bool, ...] = (), unroll_limit: int = 0):
        self.fn_name = fn_name
        self.core_num = core_num
        self.block_idx = PlainValue.sym("block_idx")
        self.loops: List[Loop] = []
        self.effects: List[Effect] = []
        self.tensors: List[Any] = []
        self._loop_ids = itertools.count()
        # ``if`` on a run-time scalar: the kernel is traced once per path.  `forced` holds the outcomes this run must
        # take at its first branches (further ones default to True); `taken` records every (condition, outcome).
        self.forced = tuple(forced)
        self.taken: List[Tuple[PlainValue, bool]] = []
        # loops with compile-time bounds and at most this many iterations are unrolled while tracing (0: never)
        self.unroll_limit = unroll_limit
        self.masks: List[Tuple[PlainValue, Optional[PlainValue]]] = []     # active ``asc2.mask`` contexts, innermost last

    # -- branches ---------------------------------------------------------------------------------
    MAX_BRANCHES = 256      # run-time conditions one trace may evaluate

    def branch(self, cond: PlainValue) -> bool:
        if len(self.taken) >= self.MAX_BRANCHES:
            # a `while` on a run-time value never ends while tracing: every evaluation is another taken branch
            raise NotImplementedError(
                f"kernel '{self.fn_name}' evaluated more than {self.MAX_BRANCHES} run-time conditions in one trace: a "
                "`while` loop on a run-time value is not supported, iterate with `for ... in asc2.range(...)`")
        outcome = self.forced[len(self.taken)] if len(self.taken) < len(self.forced) else True
        self.taken.append((cond, outcome))
        return outcome

    # -- loops ------------------------------------------------------------------------------------
    def push_loop(self, start, stop, step, unroll_factor: int, parallel: bool) -> Loop:
        var = PlainValue.sym(f"i{next(self._loop_ids)}")
        loop = Loop(var, start, stop, step, unroll_factor, parallel)
        self.loops.append(loop)
        return loop

    def pop_loop(self, loop: Loop) -> None:
        assert self.loops and self.loops[-1] is loop
        self.loops.pop()

    def loop_nest(self) -> Tuple[Loop, ...]:
        return tuple(self.loops)

    # -- recording --------------------------------------------------------------------------------
    def node(self, _kind: str, /, *args, **attrs) -> Node:
        return Node(_kind, args, attrs, self.loop_nest())

    def effect(self, _kind: str, /, *args, **attrs) -> None:
        self.effects.append(Effect(_kind, args, attrs, self.loop_nest(), tuple(self.taken)))

    def __enter__(self) -> "TraceContext":
        global _current
        if _current is not None:
            raise RuntimeError("Nested kernel tracing is not supported")
        _current = self
        return self

    def __exit__(self, *exc) -> None:
        global _current
        _current = None


def current() -> TraceContext:
    if _current is None:
        raise RuntimeError("asc2 operations can only be used inside a function decorated with @asc2.jit")
    return _current


def is_tracing() -> bool:
    return _current is not None
