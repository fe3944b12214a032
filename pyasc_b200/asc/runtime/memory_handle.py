"""How kernel arguments reach device memory
(reference: python/asc/runtime/memory_handle.py:28-125).

Host tensors (NumPy, torch CPU) get a device mirror for the duration of the launch; CUDA torch
tensors pass their ``data_ptr()`` through untouched, as NPU tensors do in the reference
(memory_handle.py:94-106)."""
from __future__ import annotations

import abc
import ctypes
from typing import Optional

import numpy

from ..lib import runtime as rt


class MemoryHandle(abc.ABC):
    nbytes: int = 0

    @abc.abstractmethod
    def copy_to_device(self, stream=None) -> int:
        raise NotImplementedError

    @abc.abstractmethod
    def copy_from_device(self, stream=None) -> None:
        raise NotImplementedError

    @abc.abstractmethod
    def release_memory(self) -> None:
        raise NotImplementedError


class _HostMirror(MemoryHandle):

    def __init__(self) -> None:
        self.handle: Optional[ctypes.c_void_p] = None

    def _host_ptr(self) -> int:
        raise NotImplementedError

    def host_ptr(self) -> int:
        return self._host_ptr()

    def is_pinned(self) -> bool:
        """True when the host buffer is page-locked, i.e. asynchronous copies really are asynchronous."""
        return False

    def copy_to_device(self, stream=None) -> int:
        self.handle = rt.copy_data_to_device(ctypes.c_void_p(self._host_ptr()), self.nbytes, stream)
        return int(self.handle.value)

    def device_alloc_only(self) -> int:
        """Device mirror without the upload (for arguments the kernel only writes)."""
        self.handle = rt.malloc(self.nbytes)
        return int(self.handle.value)

    def copy_from_device(self, stream=None) -> None:
        rt.copy_data_from_device(ctypes.c_void_p(self._host_ptr()), self.handle, self.nbytes, stream)

    def release_memory(self) -> None:
        if self.handle is not None:
            rt.free(self.handle)
            self.handle = None


class ByteArrayHandle(_HostMirror):

    def __init__(self, data):
        super().__init__()
        self.data = data if isinstance(data, bytearray) else bytearray(data)
        self._buf = (ctypes.c_char * len(self.data)).from_buffer(self.data)
        self.nbytes = len(self.data)

    def _host_ptr(self) -> int:
        return ctypes.addressof(self._buf)


class NumpyArrayHandle(_HostMirror):

    def __init__(self, array: numpy.ndarray):
        super().__init__()
        if not array.flags["C_CONTIGUOUS"]:
            raise RuntimeError("NumPy kernel arguments must be C-contiguous")
        self.array = array
        self.nbytes = array.nbytes

    def _host_ptr(self) -> int:
        return self.array.ctypes.data


class TorchCpuTensorHandle(_HostMirror):

    def __init__(self, tensor):
        super().__init__()
        if not tensor.is_contiguous():
            raise RuntimeError("torch kernel arguments must be contiguous")
        self.tensor = tensor
        self.nbytes = tensor.numel() * tensor.element_size()

    def _host_ptr(self) -> int:
        return self.tensor.data_ptr()

    def is_pinned(self) -> bool:
        try:
            return bool(self.tensor.is_pinned())
        except RuntimeError:   # no CUDA context available to ask
            return False


class TorchCudaTensorArgument(MemoryHandle):
    """Zero-copy: the tensor already lives on the device."""

    def __init__(self, tensor):
        if not tensor.is_contiguous():
            raise RuntimeError("torch kernel arguments must be contiguous")
        self.tensor = tensor
        self.nbytes = tensor.numel() * tensor.element_size()

    def copy_to_device(self, stream=None) -> int:
        return self.tensor.data_ptr()

    def copy_from_device(self, stream=None) -> None:
        pass

    def release_memory(self) -> None:
        pass


def resolve_memory_handle(obj) -> MemoryHandle:
    if isinstance(obj, MemoryHandle):
        return obj
    if isinstance(obj, (bytes, bytearray)):
        return ByteArrayHandle(obj)
    if isinstance(obj, numpy.ndarray):
        return NumpyArrayHandle(obj)
    try:
        import torch
        if isinstance(obj, torch.Tensor):
            if obj.is_cuda:
                return TorchCudaTensorArgument(obj)
            if obj.is_cpu:
                return TorchCpuTensorHandle(obj)
    except ModuleNotFoundError:
        pass
    raise RuntimeError(f"Unsupported memory handle of type {obj.__class__.__name__}")
