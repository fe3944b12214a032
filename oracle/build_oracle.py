"""Builds oracle/oracle.c into oracle/_build/liboracle.so with gcc and loads it with ctypes.
TEST INFRASTRUCTURE: used by tests/ and by bench.py's CPU-baseline leg only.

The reference itself cannot be compiled here (its hot path is lowered through MLIR into Ascend C and
built by the CANN toolkit's bisheng compiler, none of which exist on this machine), so there is no
oracle/_ref build; this C file plus oracle/golden.py stand in for it."""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path
from typing import Optional

HERE = Path(__file__).resolve().parent
SRC = HERE / "oracle.c"
OUT_DIR = HERE / "_build"
LIB = OUT_DIR / "liboracle.so"

_lib: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> Path:
    if LIB.exists() and not force and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", "-o", str(LIB), str(SRC), "-lm"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{res.stdout}")
    return LIB


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(build()))
        P = c_void_p
        lib.oracle_vadd_f32.argtypes = [P, P, P, c_int64]
        lib.oracle_vmuladd_f32.argtypes = [P, P, P, P, c_int64]
        lib.oracle_softmax_f32.argtypes = [P, P, c_int64, c_int64]
        lib.oracle_gemm_16.argtypes = [P, P, P, c_int64, c_int64, c_int64, c_int]
        lib.oracle_gemm_i8.argtypes = [P, P, P, c_int64, c_int64, c_int64]
        lib.oracle_dequant_f16.argtypes = [P, P, P, P, c_int64, c_int64]
        lib.oracle_attention_f16.argtypes = [P, P, P, P, c_int64, c_int64, c_int64, c_float, c_int]
        for name in ("oracle_vadd_f32", "oracle_vmuladd_f32", "oracle_softmax_f32", "oracle_gemm_16",
                     "oracle_gemm_i8", "oracle_dequant_f16", "oracle_attention_f16"):
            getattr(lib, name).restype = None
        _lib = lib
    return _lib


if __name__ == "__main__":
    print(build(force=True))
