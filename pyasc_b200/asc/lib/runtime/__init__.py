"""``asc.lib.runtime`` (reference: python/asc/lib/runtime/__init__.py): the functions of
:mod:`.interface` plus the handle types of :mod:`.support`."""
from .interface import *  # noqa: F401,F403
from .interface import (check_device_status, copy_data_from_device, copy_data_to_device, create_stream,  # noqa: F401
                        current_device, current_platform, current_stream, default_device, destroy_stream,
                        device_count, device_info, free, get_soc_version, is_available, is_initialized, is_model,
                        launch_count, malloc, memcpy, memcpy_async, release_pool, reset_device, set_device,
                        set_soc_version, synchronize, synchronize_device, use_cuda, use_model, use_npu)
from .support import (DeviceInfoType, DeviceModuleType, Event, MallocPolicy, Memory, MemcpyKind, MemoryType,  # noqa: F401
                      Stream)
from . import state  # noqa: F401
