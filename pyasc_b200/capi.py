"""ctypes binding of libasc_cuda.so — the one place the shared library is loaded.

Mirrors the reference's ``RuntimeInterface`` (python/asc/lib/runtime/state.py:25-75): the
library is loaded with ``ctypes.CDLL`` and every call goes through :func:`call`, which raises
``RuntimeError`` on a non-zero status.  There is no CPU fallback: when the library is missing
and cannot be built, loading raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int32, c_int64, c_uint16, c_uint32, c_uint64, c_void_p
from typing import Dict, Optional, Sequence

from . import build as _build

_lib: Optional[ctypes.CDLL] = None

P = c_void_p

# name -> argtypes; every function returns int32 status.  Kept in step with include/asc_cuda.h.
PROTOTYPES: Dict[str, Sequence] = {
    "GetSocVersionWrapper": (c_char_p, c_uint32),
    "GetDeviceCountWrapper": (P,),
    "GetDeviceInfoWrapper": (c_uint32, c_int32, c_int32, P),
    "DeviceResetWrapper": (c_int32,),
    "SetDeviceWrapper": (c_int32,),
    "StreamCreateWrapper": (P, c_int32),
    "StreamDestroyWrapper": (P,),
    "MallocWrapper": (P, c_uint64, c_int32, c_uint16),
    "MemcpyWrapper": (P, c_uint64, P, c_uint64, c_int32),
    "MemcpyAsyncWrapper": (P, c_uint64, P, c_uint64, c_int32, P),
    "StreamSynchronizeWithTimeoutWrapper": (P, c_int32),
    "StreamSynchronizeWrapper": (P,),
    "FreeWrapper": (P,),
    "DeviceSynchronizeWrapper": (),
    "HostMallocWrapper": (P, c_uint64),
    "HostFreeWrapper": (P,),
    "HostRegisterWrapper": (P, c_uint64),
    "HostUnregisterWrapper": (P,),
    "asc_cuda_event_create": (P,),
    "asc_cuda_event_create_notiming": (P,),
    "StreamWaitEventWrapper": (P, P),
    "asc_cuda_event_record": (P, P),
    "asc_cuda_event_synchronize": (P,),
    "asc_cuda_event_elapsed_ms": (P, P, P),
    "asc_cuda_event_destroy": (P,),
    "asc_cuda_status_string": (c_int32, c_char_p, c_uint32),
    "asc_cuda_last_cuda_error": (c_char_p, c_uint32),
    "asc_cuda_check_device_status": (P, P),
    "asc_cuda_launch_count": (P,),
    "asc_cuda_vadd_f32": (P, P, P, c_int64, P),
    "asc_cuda_vmuladd_f32": (P, P, P, P, c_int64, P),
    "asc_cuda_eltwise_program": (P, P, c_int32, P, P, c_int32, P, c_int32, c_int64, P),
    "asc_cuda_eltwise_program_2d": (P, P, c_int32, P, P, c_int32, P, c_int32, c_int64, c_int64, P, P),
    "asc_cuda_row_program": (P, P, c_int32, P, P, c_int32, P, c_int32, c_int64, c_int64, P, c_int32, P),
    "asc_cuda_col_program": (P, P, c_int32, P, P, c_int32, P, c_int32, c_int64, c_int64, P, c_int32, P),
    "asc_cuda_register_program": (c_int32, P, c_int32, P),
    "asc_cuda_copy_2d": (P, P, c_int64, c_int64, c_int64, c_int64, P),
    "asc_cuda_convert_bytes": (P, P, c_int64, c_int32, P),
    "asc_cuda_reduce_f32": (P, P, c_int64, c_int64, c_int64, c_int32, c_int32, c_int64, P),
    "asc_cuda_reduce_all_f16": (P, P, c_int64, c_int64, c_int64, c_int32, c_int64, c_int32, P),
    "asc_cuda_softmax_f32": (P, P, c_int64, c_int64, c_int64, P),
    "asc_cuda_softmax_f16": (P, P, c_int64, c_int64, c_int64, P),
    "asc_cuda_rms_norm_f32": (P, P, P, c_int64, c_int64, c_int64, c_float, P),
    "asc_cuda_rms_norm_f16": (P, P, P, c_int64, c_int64, c_int64, c_float, P),
    "asc_cuda_gemm_f16": (P, P, P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32,
                          c_int32, P),
    "asc_cuda_gemm_f16_bias": (P, P, P, P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32,
                               c_int32, c_int32, P),
    "asc_cuda_gemm_f16_static_workspace": (P, P, P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32,
                                           c_int32, P),
    "asc_cuda_gemm_f32": (P, P, P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, P),
    "asc_cuda_gemm_i8": (P, P, P, P, P, P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, P),
    "asc_cuda_attn_fwd_f16": (P, P, P, P, c_int32, c_int32, c_int32, c_int32, c_float, c_int32, c_int32, P),
}

# Tuning hooks (declared in include/asc_cuda_tuning.h); bound when present.
TUNING_PROTOTYPES: Dict[str, Sequence] = {
    "asc_cuda_vadd_f32_variant": (P, P, P, c_int64, c_int32, P),
    "asc_cuda_softmax_f32_variant": (P, P, c_int64, c_int64, c_int64, c_int32, P),
    "asc_cuda_gemm_capped": (P, P, P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, c_int32, P),
    "asc_cuda_gemm_set_mode": (c_int32, ),
    "asc_cuda_eltwise_set_lanes": (c_int32, ),
    "asc_cuda_selftest_wait_runs_out": (P, P),
}


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load (building first when the sources changed) and prototype the shared library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.lib_path()
    if build_if_missing and not _build.is_current():
        path = _build.build()   # a failed build raises: a stale library is never used silently
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m pyasc_b200.build` (needs nvcc); "
                           "there is no CPU fallback for the CUDA platform")
    lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    for name, argtypes in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library diverged
        fn.argtypes = list(argtypes)
        fn.restype = c_int32
    for name, argtypes in TUNING_PROTOTYPES.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = list(argtypes)
            fn.restype = c_int32
    _lib = lib
    return lib


def status_string(code: int) -> str:
    buf = ctypes.create_string_buffer(128)
    load().asc_cuda_status_string(code, buf, 128)
    return buf.value.decode()


def last_cuda_error() -> str:
    buf = ctypes.create_string_buffer(512)
    load().asc_cuda_last_cuda_error(buf, 512)
    return buf.value.decode()


def call(fn_name: str, *args) -> None:
    """Call an entry point; non-zero status -> RuntimeError (reference: state.py:64-75)."""
    fn = getattr(load(), fn_name)
    error = fn(*args)
    if error != 0:
        detail = status_string(error)
        if error == 4:
            detail += ": " + last_cuda_error()
        raise RuntimeError(f"Function {fn_name} returned {error} ({detail})")


def launch_count() -> int:
    n = c_uint64(0)
    call("asc_cuda_launch_count", ctypes.addressof(n))
    return int(n.value)


def check_device_status(stream: Optional[int] = None) -> None:
    """Synchronise ``stream`` and raise if a kernel reported a timed-out device-side wait."""
    code = c_uint32(0)
    rc = load().asc_cuda_check_device_status(stream, ctypes.addressof(code))
    if rc != 0:
        raise RuntimeError(f"device status word = {hex(code.value)} (status {rc}: {status_string(rc)})")
