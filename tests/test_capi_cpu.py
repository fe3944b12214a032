"""The C-ABI library loads without a GPU, exports every symbol include/*.h declares, and rejects bad
arguments on the host before any launch.  No compute call is made here."""
import ctypes
import glob
import os
import re

import pytest

from pyasc_b200 import build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
        names += re.findall(r"\bint32_t\s+(\w+)\s*\(", text)
    return sorted(set(names))


def test_library_builds_and_loads():
    path = build.build()
    assert path.exists()
    assert capi.load() is not None


def test_every_declared_symbol_is_exported():
    lib = capi.load()
    names = declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_every_prototype_is_declared():
    names = set(declared_symbols())
    for n in list(capi.PROTOTYPES) + list(capi.TUNING_PROTOTYPES):
        assert n in names, f"{n} is bound in capi.py but not declared in include/"


def test_status_strings():
    assert capi.status_string(0) == "ok"
    assert "misaligned" in capi.status_string(2)
    assert capi.status_string(12345) == "unknown status"


def test_bad_arguments_are_rejected_on_host():
    lib = capi.load()
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    assert lib.asc_cuda_vadd_f32(None, None, None, 16, None) == 1
    assert lib.asc_cuda_vadd_f32(p, p, p, -1, None) == 1
    assert lib.asc_cuda_vadd_f32(p, p, p, 0, None) == 0          # empty input: nothing to do
    assert lib.asc_cuda_softmax_f32(p, p, 4, 8, 4, None) == 1    # pitch smaller than the row
    assert lib.asc_cuda_softmax_f32(p, p, 0, 8, 8, None) == 0
    assert lib.asc_cuda_gemm_f16(None, p, p, 16, 16, 16, 16, 16, 16, 0, 0, 0, None) == 1
    assert lib.asc_cuda_gemm_f16(p, p, p, 16, 16, 16, 16, 16, 16, 5, 0, 0, None) == 1   # bad dtype code
    assert lib.asc_cuda_gemm_f16(p, p, p, 16, 16, 16, 16, 16, 16, 0, 0, 2, None) == 3   # accumulate needs fp32 out
    assert lib.asc_cuda_gemm_f16(p + 2, p, p, 16, 16, 16, 16, 16, 16, 0, 0, 0, None) == 2
    assert lib.asc_cuda_gemm_f16(p, p, p, 16, 16, 20, 20, 16, 16, 0, 0, 0, None) == 2   # lda * 2 not a multiple of 16
    assert lib.asc_cuda_gemm_i8(p, p, None, None, None, None, 16, 16, 16, 16, 16, 16, None) == 1
    assert lib.asc_cuda_gemm_i8(p, p, None, p, None, None, 16, 16, 16, 16, 16, 16, None) == 1  # scales missing
    assert lib.asc_cuda_attn_fwd_f16(p, p, p, p, 1, 1, 128, 64, 0.1, 0, 0, None) == 3   # head size != 128
    assert lib.asc_cuda_attn_fwd_f16(p, p, p, p, 0, 1, 128, 128, 0.1, 0, 0, None) == 1
    assert lib.MemcpyWrapper(p, 4, p, 8, 0) == 1                # more bytes than the destination holds


def test_call_raises_runtime_error_with_the_reference_message():
    with pytest.raises(RuntimeError, match=r"Function asc_cuda_vadd_f32 returned 1"):
        capi.call("asc_cuda_vadd_f32", None, None, None, 16, None)


def test_launch_counter_counts_nothing_on_cpu():
    assert capi.launch_count() >= 0
