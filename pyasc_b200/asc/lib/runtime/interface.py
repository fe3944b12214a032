"""Python face of the device runtime for the CUDA platform
(reference: python/asc/lib/runtime/interface.py:25-423): lazy initialisation, device and stream
management, malloc / memcpy / free, synchronisation.  Every function forwards to a C-ABI wrapper of
libasc_cuda.so through ``state.lib.call``.

Differences from the reference that callers can observe: device memory freed through
:func:`free` goes to a size-bucketed pool and is reused by the next :func:`malloc` of that size
(``cudaFree`` synchronises the whole device; :func:`release_pool` really frees), and
``reset_device`` destroys the streams this module created but never resets the GPU, which is
shared with other processes.
"""
from __future__ import annotations

import atexit
import ctypes
from typing import Callable, Dict, List, Optional

from . import state, support

_pool: Dict[int, List[int]] = {}
_POOL_LIMIT_BYTES = 8 << 30
_pool_bytes = 0
# callables(device_id) run by reset_device before the device's streams are destroyed, so that modules holding
# streams or events of that device (the launcher's copy/compute pipeline) can drop them
_reset_hooks: List[Callable[[int], None]] = []


def on_device_reset(hook: Callable[[int], None]) -> None:
    if hook not in _reset_hooks:
        _reset_hooks.append(hook)


def _lazy_init(need_device: bool = True, need_stream: bool = True) -> None:
    if state.lib is None:
        state.load_lib()
        atexit.register(_shutdown)
    if not need_device:
        return
    if state.device_id is None:
        set_device(default_device())
    if not need_stream:
        return
    if state.streams.get(state.device_id) is None:
        state.streams[state.device_id] = create_stream()


def _shutdown() -> None:
    try:
        release_pool()
        for handle in tuple(state.allocs.keys()):
            state.lib.call("FreeWrapper", ctypes.c_void_p(handle))
            del state.allocs[handle]
    except Exception:
        pass


def use_cuda() -> None:
    state.backend = "CUDA"


def use_model(custom_lib_prefix: Optional[str] = None) -> None:
    raise RuntimeError("The CANN simulator back end is not part of the CUDA platform build")


def use_npu(custom_lib_prefix: Optional[str] = None) -> None:
    raise RuntimeError("The Ascend NPU back end is not part of the CUDA platform build")


def set_soc_version(soc_verison) -> None:
    state.soc_verison = soc_verison


def get_soc_version():
    return state.soc_verison


def is_initialized() -> bool:
    return state.lib is not None


def is_available() -> bool:
    """True when libasc_cuda.so loads and at least one CUDA device is visible."""
    try:
        _lazy_init(need_device=False)
        return device_count() > 0
    except Exception:
        return False


def is_model() -> bool:
    return False


def check_device_handle(device_id: int) -> None:
    if isinstance(device_id, int) and device_id >= 0:
        return
    raise RuntimeError(f"Device handle should be int >= 0, but '{device_id}' with {type(device_id)} type was given")


def default_device() -> int:
    return 0


def current_device() -> int:
    _lazy_init(need_stream=False)
    return state.device_id


def current_stream(device_id: Optional[int] = None) -> support.Stream:
    _lazy_init()
    dev = state.device_id if device_id is None else device_id
    check_device_handle(dev)
    return state.streams[dev]


def current_platform() -> str:
    _lazy_init(need_device=False)
    buf = ctypes.create_string_buffer(64)
    state.lib.call("GetSocVersionWrapper", buf, ctypes.c_uint32(64))
    return buf.value.decode("utf-8")


def device_count() -> int:
    _lazy_init(need_device=False)
    count = ctypes.c_int32(0)
    try:
        state.lib.call("GetDeviceCountWrapper", ctypes.c_void_p(ctypes.addressof(count)))
    except RuntimeError:
        return 0
    return int(count.value)


def device_info(module_type: support.DeviceModuleType, info_type: support.DeviceInfoType,
                device_id: Optional[int] = None) -> int:
    _lazy_init(need_stream=False)
    dev = state.device_id if device_id is None else device_id
    result = ctypes.c_int64(0)
    state.lib.call("GetDeviceInfoWrapper", ctypes.c_uint32(dev), ctypes.c_int32(module_type.value),
                   ctypes.c_int32(info_type.value), ctypes.c_void_p(ctypes.addressof(result)))
    return int(result.value)


def reset_device(device_id: Optional[int] = None) -> None:
    if state.lib is None:
        return
    dev = state.device_id if device_id is None else device_id
    if dev is None:
        return
    release_pool()
    for hook in _reset_hooks:
        hook(dev)
    state.lib.call("DeviceResetWrapper", ctypes.c_int32(dev))
    state.streams[dev] = None
    if dev == state.device_id:
        state.device_id = None


def set_device(device_id: int) -> None:
    check_device_handle(device_id)
    _lazy_init(need_device=False)
    if state.device_id is not None and state.device_id != device_id:
        release_pool()
    state.lib.call("SetDeviceWrapper", ctypes.c_int32(device_id))
    state.device_id = device_id
    state.streams.setdefault(device_id, None)


def create_stream(priority: int = 0) -> support.Stream:
    _lazy_init(need_stream=False)
    handle = ctypes.c_void_p()
    state.lib.call("StreamCreateWrapper", ctypes.c_void_p(ctypes.addressof(handle)), ctypes.c_int32(priority))
    return handle


def destroy_stream(stream_handle: support.Stream) -> None:
    if stream_handle is None:
        return
    _lazy_init(need_stream=False)
    state.lib.call("StreamDestroyWrapper", stream_handle)


def _bucket(size: int) -> int:
    if size <= 4096:
        return 4096
    return 1 << (size - 1).bit_length() if size < (1 << 20) else ((size + (1 << 20) - 1) >> 20) << 20


def malloc(size: int, memory_type: support.MemoryType = support.MemoryType.RT_MEMORY_DEFAULT,
           policy: support.MallocPolicy = support.MallocPolicy.RT_MEMORY_POLICY_NONE) -> support.Memory:
    global _pool_bytes
    if size <= 0:
        raise RuntimeError("Malloc size must be greater than 0!")
    _lazy_init()
    real = _bucket(size)
    free_list = _pool.get(real)
    if free_list:
        ptr = free_list.pop()
        _pool_bytes -= real
    else:
        handle = ctypes.c_void_p()
        try:
            state.lib.call("MallocWrapper", ctypes.c_void_p(ctypes.addressof(handle)), ctypes.c_uint64(real),
                           ctypes.c_int32(memory_type.value | policy.value), ctypes.c_uint16(33))
        except RuntimeError:
            release_pool()
            state.lib.call("MallocWrapper", ctypes.c_void_p(ctypes.addressof(handle)), ctypes.c_uint64(real),
                           ctypes.c_int32(memory_type.value | policy.value), ctypes.c_uint16(33))
        ptr = handle.value
    state.allocs[ptr] = real
    return ctypes.c_void_p(ptr)


def free(mem_handle: support.Memory) -> None:
    global _pool_bytes
    _lazy_init(need_stream=False)
    ptr = mem_handle.value if isinstance(mem_handle, ctypes.c_void_p) else int(mem_handle)
    real = state.allocs.pop(ptr)
    if _pool_bytes + real <= _POOL_LIMIT_BYTES:
        _pool.setdefault(real, []).append(ptr)
        _pool_bytes += real
    else:
        state.lib.call("FreeWrapper", ctypes.c_void_p(ptr))


def release_pool() -> None:
    """Return every pooled device buffer to the driver."""
    global _pool_bytes
    if state.lib is None:
        return
    for free_list in _pool.values():
        for ptr in free_list:
            state.lib.call("FreeWrapper", ctypes.c_void_p(ptr))
    _pool.clear()
    _pool_bytes = 0


def memcpy(mem_dst_handle, dst_nbytes: int, mem_src_handle, src_nbytes: int, kind: support.MemcpyKind) -> None:
    if dst_nbytes <= 0 or src_nbytes <= 0:
        raise RuntimeError("Memcopy src and dst size must be greater than 0!")
    _lazy_init()
    state.lib.call("MemcpyWrapper", ctypes.cast(mem_dst_handle, ctypes.c_void_p), ctypes.c_uint64(dst_nbytes),
                   ctypes.cast(mem_src_handle, ctypes.c_void_p), ctypes.c_uint64(src_nbytes), kind.value)


def memcpy_async(mem_dst_handle, dst_nbytes: int, mem_src_handle, src_nbytes: int, kind: support.MemcpyKind,
                 stream_handle: Optional[support.Stream] = None) -> None:
    if dst_nbytes <= 0 or src_nbytes <= 0:
        raise RuntimeError("Memcopy src and dst size must be greater than 0!")
    _lazy_init()
    if stream_handle is None:
        stream_handle = current_stream()
    state.lib.call("MemcpyAsyncWrapper", ctypes.cast(mem_dst_handle, ctypes.c_void_p), ctypes.c_uint64(dst_nbytes),
                   ctypes.cast(mem_src_handle, ctypes.c_void_p), ctypes.c_uint64(src_nbytes), kind.value,
                   stream_handle)


def copy_data_to_device(src_mem_handle, nbytes: int, stream_handle: Optional[support.Stream] = None) -> support.Memory:
    dst = malloc(nbytes, support.MemoryType.RT_MEMORY_HBM)
    memcpy_async(dst, nbytes, src_mem_handle, nbytes, support.MemcpyKind.RT_MEMCPY_HOST_TO_DEVICE, stream_handle)
    return dst


def copy_data_from_device(mem_dst_handle, mem_src_handle, nbytes: int,
                          stream_handle: Optional[support.Stream] = None) -> None:
    memcpy_async(mem_dst_handle, nbytes, mem_src_handle, nbytes, support.MemcpyKind.RT_MEMCPY_DEVICE_TO_HOST,
                 stream_handle)


def synchronize(stream_handle: Optional[support.Stream] = None, timeout: int = 0) -> None:
    _lazy_init()
    if stream_handle is None:
        stream_handle = current_stream()
    if timeout > 0:
        state.lib.call("StreamSynchronizeWithTimeoutWrapper", stream_handle, ctypes.c_int32(timeout))
    else:
        state.lib.call("StreamSynchronizeWrapper", stream_handle)


def synchronize_device() -> None:
    _lazy_init()
    state.lib.call("DeviceSynchronizeWrapper")


def check_device_status(stream_handle: Optional[support.Stream] = None) -> None:
    """Synchronise and raise if a kernel gave up on a bounded device-side wait."""
    _lazy_init()
    if stream_handle is None:
        stream_handle = current_stream()
    code = ctypes.c_uint32(0)
    try:
        state.lib.call("asc_cuda_check_device_status", stream_handle, ctypes.c_void_p(ctypes.addressof(code)))
    except RuntimeError as e:
        raise RuntimeError(f"{e}; device status word {hex(code.value)}") from None


def launch_count() -> int:
    _lazy_init(need_device=False)
    n = ctypes.c_uint64(0)
    state.lib.call("asc_cuda_launch_count", ctypes.c_void_p(ctypes.addressof(n)))
    return int(n.value)
