"""``asc``: the part of PyAsc's top-level package that asc2 scripts use, on the CUDA platform
(reference: python/asc/__init__.py)."""
import os as _os
import sys as _sys

# `pyasc_b200` (the ctypes binding and build of libasc_cuda) must be importable next to this package
_repo_root = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _repo_root not in _sys.path:
    _sys.path.append(_repo_root)

from .language import *  # noqa: F401,F403,E402
from .language import __all__ as _lan_all  # noqa: E402
from .runtime.options import CodegenOptions, CompileOptions, LaunchOptions  # noqa: E402
from .runtime.jit import jit  # noqa: E402
from . import lib, runtime, language  # noqa: F401,E402

__all__ = ["CodegenOptions", "CompileOptions", "jit", "LaunchOptions"]
__all__.extend(_lan_all)
