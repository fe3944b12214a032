"""``asc2.jit`` (reference: python/asc2/jit.py:29-52): ``asc.runtime.jit.JITFunction`` with the
asc2 defaults — ``range`` inside the kernel is ``asc2.range``; the Ascend pass-pipeline switches
are accepted for compatibility."""
from typing import Callable, Optional

from asc.language.tile.range import range as asc2_range
from asc.runtime.jit import JITFunction


def jit(fn: Optional[Callable] = None, **options):
    options.setdefault("custom_builtins", {"range": asc2_range})
    options.setdefault("insert_sync", True)
    options.setdefault("run_asc2_passes", True)

    def decorator(fn: Callable) -> JITFunction:
        return JITFunction(fn, **options)

    if fn is None:
        return decorator
    return decorator(fn)
