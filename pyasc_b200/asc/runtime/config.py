"""Platform selection (reference: python/asc/runtime/config.py:15-101).

The CUDA platform is a third ``Backend`` member and ``B200`` a ``Platform`` member; the Ascend
members stay so that scripts and test fixtures that name them still import, but selecting them
raises because this build ships no Ascend back end.
"""
from enum import Enum
from typing import Optional, Union

from ..lib import runtime as rt


class Backend(Enum):
    Model = "Model"
    NPU = "NPU"
    CUDA = "CUDA"


class Platform(Enum):
    Ascend910B1 = "Ascend910B1"
    Ascend910B2 = "Ascend910B2"
    Ascend910B3 = "Ascend910B3"
    Ascend910B4 = "Ascend910B4"
    Ascend910_9391 = "Ascend910_9391"
    Ascend910_9599 = "Ascend910_9599"
    Ascend950PR_9599 = "Ascend950PR_9599"
    B200 = "B200"


class CompilationArch(Enum):
    C220 = "c220"
    C310 = "c310"
    SM100A = "sm_100a"

    def __str__(self) -> str:
        return self.value


class KernelType(Enum):
    AIV_ONLY = 0
    AIC_ONLY = 1
    MIX_AIV_HARD_SYNC = 2
    MIX_AIC_HARD_SYNC = 3
    MIX_AIV_1_0 = 4
    MIX_AIC_1_0 = 5
    MIX_AIC_1_1 = 6
    MIX_AIC_1_2 = 7


def set_platform(
    backend: Union[Backend, str],
    soc_version: Optional[Platform] = None,
    device_id: Optional[int] = None,
    check=True,
) -> None:
    """Select the runtime back end and device.  For ``Backend.CUDA`` the SoC argument is accepted
    for signature compatibility; any value other than ``None`` / ``Platform.B200`` is ignored with
    the platform set to B200, because existing test fixtures pass an Ascend default."""
    backend = Backend(backend)
    if backend == Backend.CUDA:
        rt.use_cuda()
        soc_version = Platform.B200
    elif backend in (Backend.Model, Backend.NPU):
        raise ValueError(f"Execution backend {backend.value} is not available in the CUDA platform build; "
                         "use set_platform('CUDA')")
    else:
        raise ValueError(f"Unknown execution backend: {backend}")
    rt.set_soc_version(soc_version)
    if device_id is not None:
        if rt.state.device_id != device_id:
            rt.set_device(device_id)
    if check and not rt.is_available():
        raise RuntimeError("Runtime library is not available! libasc_cuda.so could not be loaded or no CUDA "
                           "device is visible")


def platform_to_arch(platform: Union[Platform, str]) -> CompilationArch:
    platform_name = Platform(platform).value
    if platform_name == "B200":
        return CompilationArch.SM100A
    if platform_name.startswith("Ascend910B") or platform_name.startswith("Ascend910_93"):
        return CompilationArch.C220
    if platform_name.startswith("Ascend910_95") or platform_name.startswith("Ascend950PR_95"):
        return CompilationArch.C310
    raise ValueError(f"There is no compilation arch for '{platform_name}' platform")
