"""``JITFunction``: what ``@asc2.jit`` returns (reference: python/asc/runtime/jit.py:33-223).

Same call shape as the reference — ``kernel[core_num](...)`` or ``kernel[core_num, stream](...)``,
option keywords from the three option dataclasses accepted at decoration and call time, ConstExpr
parameters split from run-time ones — but the body behind ``_run`` is: trace the kernel once
(:mod:`asc.codegen.tracer`), match it to CUDA kernels (:mod:`asc.codegen.matcher`), launch
(:mod:`asc.runtime.launcher`).  Plans are cached per (options, ConstExpr values, argument kinds and
shapes, scalar values, core_num); ``always_compile=True`` re-traces on every call.
"""
from __future__ import annotations

import inspect
import os
import sys
from dataclasses import fields
from typing import Any, Callable, Dict, List, Optional, Tuple, Type, Union, get_args, get_origin

import numpy as np

from ..codegen.function import Function, P, T, get_annotations
from ..language.core.constexpr import ConstExpr, require_constexpr
from ..codegen.matcher import Plan, build_plan
from ..codegen.tracer import trace_kernel
from ..language.core.dtype import DataType, KnownTypes as KT
from ..language.tile.range import range as asc2_range
from .launcher import Launcher
from .options import CodegenOptions, CompileOptions, LaunchOptions


class PlainArgType:

    def __init__(self, dtype: DataType):
        self.dtype = dtype


class PointerArgType:

    def __init__(self, dtype: DataType):
        self.dtype = dtype


UNROLL_LIMIT = 64      # iterations up to which a compile-time loop is unrolled when a tile is carried across it


class JITFunction(Function[P, T]):
    launcher: Type[Launcher] = Launcher

    def __init__(self, fn: Callable[P, T], **options):
        super().__init__(fn)
        clashed_args = self.get_clashed_args(fn)
        if clashed_args:
            raise RuntimeError("The following argument names conflict with JIT configuration options: " +
                               ", ".join(clashed_args))
        unknown_options = set(options).difference(self.get_config_keywords())
        if unknown_options:
            raise RuntimeError("The following option names are unknown: " + ", ".join(unknown_options))
        self.default_options: Dict[str, Any] = options
        self.launch_options = LaunchOptions()
        self.kernel_cache: Dict[Any, Plan] = {}
        self.last_plan: Optional[Plan] = None
        # the function's signature and annotations do not change between launches: looked up at the first one (string
        # annotations may name things that are defined after the decorator has run)
        self._signature: Optional[inspect.Signature] = None
        self._constexpr_args: Dict[str, tuple] = {}      # ConstExpr-annotated parameter -> the types it accepts

    def _bind(self, args: tuple, kwargs: Dict[str, Any]) -> Dict[str, Any]:
        if self._signature is None:
            for name, ann in get_annotations(self.fn).items():
                origin = get_origin(ann) or ann
                if isinstance(origin, type) and issubclass(origin, ConstExpr):
                    self._constexpr_args[name] = get_args(ann)
            self._signature = inspect.signature(self.fn)
        return self._signature.bind(*args, **kwargs).arguments

    def __getitem__(self, user_launch_options: Union[int, tuple]) -> Callable:
        try:
            if isinstance(user_launch_options, int):
                self.launch_options = LaunchOptions(core_num=user_launch_options)
            else:
                self.launch_options = LaunchOptions(*user_launch_options)
        except Exception as e:
            raise TypeError("Parse user launch options failed") from e
        else:
            return self._run

    @staticmethod
    def get_clashed_args(fn: Callable) -> List[str]:
        keywords = set(__class__.get_config_keywords())
        keywords.intersection_update(inspect.signature(fn).parameters)
        return list(keywords)

    @staticmethod
    def get_arg_type(value: Any):
        """Argument kind (reference: jit.py:70-96)."""
        if isinstance(value, bool):
            return PlainArgType(KT.bool_)
        if isinstance(value, int):
            return PlainArgType(KT.int_)
        if isinstance(value, float):
            return PlainArgType(KT.float_)
        if isinstance(value, np.ndarray):
            return PointerArgType(DataType(str(np.dtype(value.dtype))))
        if isinstance(value, np.generic):
            return PlainArgType(DataType(str(value.dtype)))
        try:
            import torch
            if isinstance(value, torch.Tensor):
                dtype = DataType(str(value.dtype))
                return PlainArgType(dtype) if value.dim() == 0 else PointerArgType(dtype)
        except ModuleNotFoundError:
            pass
        raise TypeError(f"Argument type in JIT function is not supported: {value.__class__.__name__}")

    _field_names: Dict[Type, Tuple[str, ...]] = {}

    @staticmethod
    def extract_kwargs(dataclass: Type, base_kwargs: Dict[str, Any]) -> Any:
        names = JITFunction._field_names.get(dataclass)
        if names is None:
            names = JITFunction._field_names[dataclass] = tuple(f.name for f in fields(dataclass))
        kwargs = {}
        for name in names:
            if name in base_kwargs:
                kwargs[name] = base_kwargs.pop(name)
        return dataclass(**kwargs)

    @classmethod
    def get_config_keywords(cls) -> List[str]:
        cached = getattr(cls, "_config_keywords", None)
        if cached is not None:
            return cached
        keywords: List[str] = []
        for dataclass in CodegenOptions, CompileOptions, LaunchOptions:
            keywords.extend(f.name for f in fields(dataclass))
        cls._config_keywords = keywords
        return keywords

    @staticmethod
    def _arg_signature(value: Any) -> Tuple:
        """What about a run-time argument shapes the plan: kind, dtype, element count, scalar value."""
        if isinstance(value, (bool, int, float)):
            return ("s", type(value).__name__, value)
        if isinstance(value, np.generic):
            return ("s", str(value.dtype), value.item())
        if isinstance(value, np.ndarray):
            return ("p", str(value.dtype), int(value.size))
        try:
            import torch
            if isinstance(value, torch.Tensor):
                if value.dim() == 0:
                    return ("s", str(value.dtype), value.item())
                return ("p", str(value.dtype), int(value.numel()))
        except ModuleNotFoundError:
            pass
        raise TypeError(f"Argument type in JIT function is not supported: {value.__class__.__name__}")

    def _cache_kernel(self, runtime_args: Dict[str, Any], constexprs: Dict[str, Any], codegen_options: CodegenOptions,
                      compile_options: CompileOptions) -> Plan:
        for value in runtime_args.values():
            self.get_arg_type(value)  # TypeError for unsupported arguments, as in the reference
        try:
            key = (self.launch_options.core_num, tuple((k, repr(v)) for k, v in constexprs.items()),
                   tuple((k, ) + self._arg_signature(v) for k, v in runtime_args.items()))
            hash(key)
        except TypeError:
            raise
        enable_cache = not compile_options.always_compile
        if enable_cache and key in self.kernel_cache:
            return self.kernel_cache[key]
        builtins = dict(codegen_options.custom_builtins) or {"range": asc2_range}
        trace = trace_kernel(self.fn, runtime_args, constexprs, self.launch_options.core_num, builtins)
        try:
            plan = build_plan(trace)
        except NotImplementedError as first:
            if "carried across iterations" not in str(first):
                raise
            # A tile flows from one loop iteration to the next (`acc = acc + tile`; the reference compiles it as
            # scf.for iteration arguments, python/asc/codegen/function_visitor.py:509-547).  A loop body traced once
            # cannot express that; with the kernel's short compile-time loops unrolled it is ordinary data flow.
            trace = trace_kernel(self.fn, runtime_args, constexprs, self.launch_options.core_num, builtins,
                                 unroll_limit=UNROLL_LIMIT)
            try:
                plan = build_plan(trace)
            except NotImplementedError:
                raise first from None
        if enable_cache:
            self.kernel_cache[key] = plan
        return plan

    def explain(self, plan: Optional[Plan] = None) -> str:
        """What a launch of this kernel runs: the recognised pattern, the library calls in order, the temporaries."""
        plan = plan if plan is not None else self.last_plan
        if plan is None:
            return f"kernel '{self.fn_name}': not launched yet"
        lines = [f"kernel '{self.fn_name}' -> {plan.pattern}: {len(plan.steps)} call(s), reads arguments "
                 f"{sorted(plan.reads, key=str)}, writes {sorted(plan.writes, key=str)}"]
        lines += [f"  temporary {k}: {v} bytes" for k, v in plan.temps.items()]
        shown = plan.steps if len(plan.steps) <= 16 else plan.steps[:8] + plan.steps[-4:]
        for i, step in enumerate(shown):
            if len(plan.steps) > 16 and i == 8:
                lines.append(f"  ... {len(plan.steps) - 12} more ...")
            lines.append(f"  {step.fn_name}: {step.note}")
        return "\n".join(lines)

    def _run(self, *args: P.args, **kwargs: P.kwargs) -> None:
        merged = dict(self.default_options)
        merged.update(kwargs)
        codegen_options = self.extract_kwargs(CodegenOptions, merged)
        compile_options = self.extract_kwargs(CompileOptions, merged)
        if self.launch_options.core_num <= 0:
            raise ValueError("Core number should be large than 0")
        call_args = self._bind(args, merged)
        # (split_args with the annotation look-ups done once, in __init__)
        runtime_args: Dict[str, Any] = {}
        constexprs: Dict[str, ConstExpr] = {}
        for name, value in call_args.items():
            accepted = self._constexpr_args.get(name)
            if accepted is None:
                runtime_args[name] = value
            else:
                if accepted:
                    require_constexpr(value, *accepted, arg_name=name)
                constexprs[name] = ConstExpr(value)
        plan = self._cache_kernel(runtime_args, constexprs, codegen_options, compile_options)
        self.last_plan = plan
        if compile_options.print_ir_before_all or os.environ.get("ASC_CUDA_EXPLAIN"):
            # the reference prints its IR here (print_ir_before_all, python/asc/runtime/compiler.py); this platform's
            # counterpart of the IR is the plan: the library calls the launch is made of
            print(self.explain(plan), file=sys.stderr)
        self.launcher(self.launch_options).run(plan, self.fn_name, tuple(runtime_args.values()))


def jit(fn: Optional[Callable[P, T]] = None, **options):
    """``asc.jit``: decorator form with or without options (reference: jit.py:240-249)."""
    from ..language.tile.range import range as default_range
    options.setdefault("custom_builtins", {"range": default_range})

    def decorator(fn: Callable[P, T]) -> JITFunction[P, T]:
        return JITFunction(fn, **options)

    if fn is None:
        return decorator
    return decorator(fn)
