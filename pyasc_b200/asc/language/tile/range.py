"""``asc2.range``: the loop construct of asc2 kernels
(reference: python/asc/language/tile/range.py:16-36, python/asc/language/core/range.py:15-89).

While a kernel is traced, iterating an ``asc2.range`` runs the loop body exactly once with a
symbolic induction variable and records the loop bounds; ``unroll_factor`` and ``parallel`` are
performance hints of the Ascend pipeline and are kept only as annotations.
"""
from __future__ import annotations

from ..core.ir_value import PlainValue
from . import trace


class range:  # noqa: A001 - mirrors the reference's name

    def __init__(self, *args, unroll_factor: int = 1, parallel: bool = False):
        if not isinstance(unroll_factor, int) or isinstance(unroll_factor, bool):
            raise TypeError(f"'unroll_factor' must be int, got {type(unroll_factor).__name__}")
        if not isinstance(parallel, bool):
            raise TypeError(f"'parallel' must be bool, got {type(parallel).__name__}")
        if unroll_factor < 1:
            raise ValueError(f"Loop unroll factor must be 1 or greater, got {unroll_factor}")
        if len(args) == 1:
            start, stop, step = 0, args[0], 1
        elif len(args) == 2:
            start, stop, step = args[0], args[1], 1
        elif len(args) == 3:
            start, stop, step = args
        else:
            raise TypeError(f"range expected 1 to 3 positional arguments, got {len(args)}")
        self.start, self.stop, self.step = start, stop, step
        self.unroll_factor = unroll_factor
        self.parallel = parallel

    def __iter__(self):
        if not trace.is_tracing():
            # outside a kernel behave like the builtin
            import builtins
            yield from builtins.range(int(self.start), int(self.stop), int(self.step))
            return
        ctx = trace.current()
        step = PlainValue.wrap(self.step)
        if step.is_const and step.value <= 0:
            raise ValueError("asc2.range requires a positive step")
        start, stop = PlainValue.wrap(self.start), PlainValue.wrap(self.stop)
        if start.is_const and stop.is_const and step.is_const and start.value >= stop.value:
            return  # statically empty loop: the body is never traced
        if ctx.unroll_limit > 0 and start.is_const and stop.is_const and step.is_const:
            import builtins
            values = builtins.range(int(start.value), int(stop.value), int(step.value))
            if len(values) <= ctx.unroll_limit:
                # unrolled trace: every iteration records its own operations, so a tile carried from one iteration
                # to the next (the reference's scf.for iteration arguments) is an ordinary value
                for i in values:
                    yield PlainValue.const(i)
                return
        loop = ctx.push_loop(self.start, self.stop, self.step, self.unroll_factor, self.parallel)
        try:
            yield loop.var
        finally:
            ctx.pop_loop(loop)


def static_range(*args):
    """Loop unrolled while tracing (reference: python/asc/language/core/range.py static_range)."""
    import builtins
    return builtins.range(*[int(a) for a in args])
