"""Process-wide state of the runtime binding (reference: python/asc/lib/runtime/state.py:25-144).

``RuntimeInterface`` owns the ``ctypes.CDLL`` of libasc_cuda.so; ``call`` raises ``RuntimeError``
on a non-zero status exactly like the reference (state.py:64-75)."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional


class RuntimeInterface:

    def __init__(self) -> None:
        from pyasc_b200 import capi
        self._capi = capi
        self.lib: ctypes.CDLL = capi.load()

    @staticmethod
    def check_error(error: int, fn_name: str) -> None:
        if error != 0:
            raise RuntimeError(f"Function {fn_name} returned {error}")

    def call(self, fn_name: str, *args) -> None:
        self._capi.call(fn_name, *args)


lib: Optional[RuntimeInterface] = None
backend: Optional[str] = None          # "CUDA" once selected
soc_verison = None                     # spelling follows the reference's attribute name
device_id: Optional[int] = None
streams: Dict[int, Optional[ctypes.c_void_p]] = {}
allocs: Dict[int, int] = {}            # user handle -> size in bytes


def load_lib() -> RuntimeInterface:
    global lib
    if lib is None:
        lib = RuntimeInterface()
    return lib
