"""Handle types and enums of the runtime binding
(reference: python/asc/lib/runtime/support.py)."""
import ctypes
import enum

Stream = ctypes.c_void_p
Memory = ctypes.c_void_p
Event = ctypes.c_void_p


class MemcpyKind(enum.Enum):
    RT_MEMCPY_HOST_TO_HOST = 0
    RT_MEMCPY_HOST_TO_DEVICE = 1
    RT_MEMCPY_DEVICE_TO_HOST = 2
    RT_MEMCPY_DEVICE_TO_DEVICE = 3


class MemoryType(enum.Enum):
    RT_MEMORY_DEFAULT = 0
    RT_MEMORY_HBM = 2


class MallocPolicy(enum.Enum):
    RT_MEMORY_POLICY_NONE = 0x0
    RT_MEMORY_POLICY_HUGE_PAGE_ONLY = 0x800


class DeviceModuleType(enum.Enum):
    RT_MODULE_TYPE_SYSTEM = 0
    RT_MODULE_TYPE_AICORE = 4  # on the CUDA platform: the SMs


class DeviceInfoType(enum.Enum):
    """infoType values understood by GetDeviceInfoWrapper of libasc_cuda."""
    INFO_TYPE_CORE_NUM = 0
    INFO_TYPE_HBM_BYTES = 1
    INFO_TYPE_L2_BYTES = 2
    INFO_TYPE_MAX_CLOCK_KHZ = 3
    INFO_TYPE_COMPUTE_CAPABILITY = 4
