"""pyasc_b200 — a CUDA (sm_100a / B200) platform behind PyAsc's asc2 operator surface.

Importing this package makes the drop-in ``asc`` and ``asc2`` packages importable (they live inside
this package directory, the way the reference keeps them under ``python/``), so an existing asc2
script only needs ``import pyasc_b200`` (or ``PYTHONPATH=<repo>/pyasc_b200``) and
``asc.runtime.config.set_platform("CUDA")``.
"""
import os as _os
import sys as _sys

_PKG_DIR = _os.path.dirname(_os.path.abspath(__file__))
if _PKG_DIR not in _sys.path:
    _sys.path.insert(0, _PKG_DIR)

__version__ = "0.1.0"
