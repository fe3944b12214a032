"""Option dataclasses whose field names are legal ``@jit(...)`` / call keywords
(reference: CodegenOptions python/asc/codegen/function_visitor.py:35-52, CompileOptions
python/asc/runtime/compiler.py:28-116, LaunchOptions python/asc/runtime/launcher.py:79-102).
The Ascend-pipeline options are accepted and ignored by the CUDA platform so that existing
scripts keep working; only ``always_compile`` (re-trace on every call) has an effect."""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class CodegenOptions:
    capture_exceptions: bool = True
    ir_multithreading: bool = True
    custom_builtins: Dict[str, Any] = field(default_factory=dict)


@dataclass
class CompileOptions:
    debug: bool = False
    strip_loc: bool = False
    verify_sync: bool = False
    print_ir_before_all: bool = False
    run_passes: bool = True
    kernel_type: Optional[Any] = None
    auto_sync: Optional[bool] = True
    auto_sync_log: Optional[str] = ""
    matmul_cube_only: bool = False
    always_compile: bool = False
    bisheng_options: Optional[Tuple[str]] = None
    opt_level: int = 3
    run_asc2_passes: bool = False
    densify_load_store: bool = False
    insert_sync: Optional[bool] = None
    reuse_ub: bool = False
    reuse_ub_in_out: bool = False
    static_alloc: Optional[bool] = None
    vf_fusion: bool = False
    common_arch: Optional[str] = None
    vec_arch: Optional[str] = None
    cube_arch: Optional[str] = None
    common_options: List[str] = field(default_factory=list)
    vec_options: List[str] = field(default_factory=list)
    cube_options: List[str] = field(default_factory=list)


@dataclass(frozen=True)
class LaunchOptions:
    core_num: int = 0
    stream: Optional[Any] = None
