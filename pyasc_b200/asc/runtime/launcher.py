"""Runs a matched kernel plan on the device (reference: python/asc/runtime/launcher.py:80-238).

Argument handling follows the reference launcher: host tensors (NumPy / torch CPU) get device
mirrors for the duration of the call and are copied back afterwards, device tensors pass through
untouched, and the call returns only after the stream has drained, so results are visible to the
caller on return.  Differences, all invisible in results: only arguments the kernel reads (or overwrites
only in part) are uploaded and only arguments it writes are copied back (the reference moves every argument both
ways, launcher.py:176-195); device mirrors come from a pool instead of malloc/free per call; and
when the caller passes its own stream (``kernel[cores, stream]``) and every argument already
lives on the device, the launch is left asynchronous on that stream.  Large launches whose host
arguments are page-locked are software-pipelined: the plan is cut into chunks along its independent
axis and upload, kernel and download of neighbouring chunks overlap on three streams, which roughly
halves the PCIe-bound end-to-end time.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np

from ..codegen.matcher import Plan
from ..lib import runtime as rt
from .memory_handle import MemoryHandle, TorchCudaTensorArgument, _HostMirror, resolve_memory_handle
from .options import LaunchOptions


PIPELINE_MIN_BYTES = 16 << 20     # below this a launch is latency-bound and is not chunked
PIPELINE_MAX_CHUNKS = int(os.environ.get("ASC_CUDA_PIPELINE_CHUNKS", "8"))

# per device: the three pipeline streams and a pool of events created on that device
_pipe_streams: Dict[int, Tuple[ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]] = {}
_event_pool: Dict[int, List[ctypes.c_void_p]] = {}


def _forget_device(dev: int) -> None:
    """``reset_device`` destroys every stream the runtime created on ``dev``: drop the handles kept here and
    destroy the device's pooled events, so the next pipelined launch makes fresh ones."""
    _pipe_streams.pop(dev, None)
    for ev in _event_pool.pop(dev, []):
        try:
            rt.state.lib.call("asc_cuda_event_destroy", ev)
        except RuntimeError:
            pass


def _pipeline_streams() -> Tuple[ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]:
    dev = rt.current_device()
    if dev not in _pipe_streams:
        rt.on_device_reset(_forget_device)
        _pipe_streams[dev] = (rt.create_stream(), rt.create_stream(), rt.create_stream())
    return _pipe_streams[dev]


def _new_event() -> ctypes.c_void_p:
    pool = _event_pool.setdefault(rt.current_device(), [])
    if pool:
        return pool.pop()
    ev = ctypes.c_void_p()
    rt.state.lib.call("asc_cuda_event_create_notiming", ctypes.c_void_p(ctypes.addressof(ev)))
    return ev


def _torch_current_stream() -> Optional[ctypes.c_void_p]:
    try:
        import torch
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)      # the handle without a Stream object around it
        if raw is not None:
            return ctypes.c_void_p(raw(torch.cuda.current_device()))
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    except Exception:
        return None


class Launcher:

    def __init__(self, options: LaunchOptions):
        self.options = options

    @staticmethod
    def get_core_num(device_id: Optional[int] = None) -> int:
        return rt.device_info(rt.DeviceModuleType.RT_MODULE_TYPE_AICORE, rt.DeviceInfoType.INFO_TYPE_CORE_NUM,
                              device_id)

    @staticmethod
    def is_scalar(value: Any) -> bool:
        if isinstance(value, (bool, int, float, np.generic)):
            return True
        try:
            import torch
            return isinstance(value, torch.Tensor) and value.dim() == 0
        except ModuleNotFoundError:
            return False

    def run(self, plan: Plan, function_name: str, user_args: Tuple[Any, ...]) -> None:
        if self.options.core_num <= 0:
            raise ValueError("Core number should be large than 0")
        if os.environ.get("DRY_RUN"):
            return
        from pyasc_b200 import jit
        jit.prepare(plan)           # expressions met for the first time get their specialised kernel built
        handles: Dict[int, MemoryHandle] = {}
        for index, arg in enumerate(user_args):
            if self.is_scalar(arg):
                continue
            try:
                handles[index] = resolve_memory_handle(arg)
            except RuntimeError as e:
                raise TypeError(f"Unsupported kernel argument of type {type(arg)}") from e
        if not plan.steps:
            return                  # no block has a tile inside its tensors (empty tensors): nothing is written
        all_on_device = all(isinstance(h, TorchCudaTensorArgument) for h in handles.values())
        self._check_device_aliasing(plan, handles)
        user_stream = self.options.stream
        if user_stream is not None:
            stream = user_stream if isinstance(user_stream, ctypes.c_void_p) else ctypes.c_void_p(int(user_stream))
        elif any(isinstance(h, TorchCudaTensorArgument) for h in handles.values()):
            # stay ordered with the torch work that produced / will consume the device tensors
            stream = _torch_current_stream() or rt.current_stream()
        else:
            stream = rt.current_stream()

        if user_stream is None and self._pipeline_applies(plan, handles):
            self._run_pipelined(plan, handles)
            return

        ptrs: Dict[Any, int] = {}
        temps: List[ctypes.c_void_p] = []
        try:
            for index, handle in handles.items():
                if isinstance(handle, _HostMirror) and index not in plan.reads and index not in plan.partial_writes:
                    ptrs[index] = handle.device_alloc_only()
                else:
                    ptrs[index] = handle.copy_to_device(stream)
            for key, nbytes in plan.temps.items():
                mem = rt.malloc(nbytes)
                temps.append(mem)
                ptrs[key] = int(mem.value)
            for step in plan.steps:
                rt.state.lib.call(step.fn_name, *step.build(ptrs, stream))
            for index, handle in handles.items():
                if index in plan.writes:
                    handle.copy_from_device(stream)
            if not (all_on_device and user_stream is not None):
                rt.check_device_status(stream)
        finally:
            if temps or not all_on_device:
                # buffers go back to the pool only once nothing on the stream can still touch them
                try:
                    rt.synchronize(stream)
                except RuntimeError:
                    pass
            for handle in handles.values():
                handle.release_memory()
            for mem in temps:
                rt.free(mem)

    # Patterns whose kernels read everything an output element depends on (its own position, or its own row held in
    # registers) before they write it: an output argument may be the very buffer of an input argument.
    _IN_PLACE_PATTERNS = ("elementwise", "softmax", "rms_norm", "row")

    @classmethod
    def _check_device_aliasing(cls, plan: Plan, handles: Dict[int, MemoryHandle]) -> None:
        """Two kernel arguments that are views of one device buffer.  Host arguments get a device buffer each, so
        they never alias; device tensors are used where they lie.  The planner reasons per argument: it cannot see
        that the matrix a GEMM stores is also the matrix its other tiles are still reading."""
        dev = {i: (h.tensor.data_ptr(), h.nbytes) for i, h in handles.items()
               if isinstance(h, TorchCudaTensorArgument) and h.nbytes}
        for w in plan.writes:
            if w not in dev:
                continue
            w_ptr, w_bytes = dev[w]
            for i, (ptr, nbytes) in dev.items():
                if i == w or (i not in plan.reads and i not in plan.writes):
                    continue
                if ptr >= w_ptr + w_bytes or w_ptr >= ptr + nbytes:
                    continue
                same = (ptr, nbytes) == (w_ptr, w_bytes) and i not in plan.writes
                if same and all(part.startswith(cls._IN_PLACE_PATTERNS) for part in plan.pattern.split("+")):
                    continue
                raise ValueError(f"Kernel arguments {i} and {w} overlap in device memory and argument {w} is written by "
                                 f"a '{plan.pattern}' launch, whose tiles run concurrently; pass separate buffers")

    # ------------------------------------------------------------------------------------------
    # chunked launch: upload / kernel / download of neighbouring chunks overlap
    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _pipeline_applies(plan: Plan, handles: Dict[int, MemoryHandle]) -> bool:
        spec = plan.pipeline
        if spec is None or os.environ.get("ASC_CUDA_NO_PIPELINE"):
            return False
        if not handles or not all(isinstance(h, _HostMirror) and h.is_pinned() for h in handles.values()):
            return False
        if not (set(handles) <= set(spec.streamed) | spec.resident):
            return False
        streamed_bytes = sum(bpu * spec.units for bpu in spec.streamed.values())
        return streamed_bytes >= PIPELINE_MIN_BYTES and spec.units >= 2 * spec.granule

    def _run_pipelined(self, plan: Plan, handles: Dict[int, MemoryHandle]) -> None:
        spec = plan.pipeline
        call = rt.state.lib.call
        s_up, s_run, s_down = _pipeline_streams()
        h2d, d2h = rt.MemcpyKind.RT_MEMCPY_HOST_TO_DEVICE, rt.MemcpyKind.RT_MEMCPY_DEVICE_TO_HOST
        granules = -(-spec.units // spec.granule)
        n_chunks = max(1, min(PIPELINE_MAX_CHUNKS, granules))
        per = -(-granules // n_chunks) * spec.granule
        bounds = [(lo, min(lo + per, spec.units)) for lo in range(0, spec.units, per)]
        ptrs: Dict[Any, int] = {}
        events: List[ctypes.c_void_p] = []
        dev = rt.current_device()
        try:
            for index, handle in handles.items():
                ptrs[index] = handle.device_alloc_only()
            for index in spec.resident:
                if index in plan.reads:
                    h = handles[index]
                    rt.memcpy_async(ctypes.c_void_p(ptrs[index]), h.nbytes, ctypes.c_void_p(h.host_ptr()), h.nbytes,
                                    h2d, s_up)
            for lo, hi in bounds:
                for index, bpu in spec.streamed.items():
                    if index in plan.reads:
                        off, n = lo * bpu, (hi - lo) * bpu
                        rt.memcpy_async(ctypes.c_void_p(ptrs[index] + off), n,
                                        ctypes.c_void_p(handles[index].host_ptr() + off), n, h2d, s_up)
                uploaded = _new_event()
                events.append(uploaded)
                call("asc_cuda_event_record", uploaded, s_up)
                call("StreamWaitEventWrapper", s_run, uploaded)
                for step in spec.make_steps(lo, hi):
                    call(step.fn_name, *step.build(ptrs, s_run))
                computed = _new_event()
                events.append(computed)
                call("asc_cuda_event_record", computed, s_run)
                call("StreamWaitEventWrapper", s_down, computed)
                for index, bpu in spec.streamed.items():
                    if index in plan.writes:
                        off, n = lo * bpu, (hi - lo) * bpu
                        rt.memcpy_async(ctypes.c_void_p(handles[index].host_ptr() + off), n,
                                        ctypes.c_void_p(ptrs[index] + off), n, d2h, s_down)
            rt.synchronize(s_down)
            rt.check_device_status(s_run)
        finally:
            for stream in (s_up, s_run, s_down):
                try:
                    rt.synchronize(stream)
                except RuntimeError:
                    pass
            _event_pool.setdefault(dev, []).extend(events)
            for handle in handles.values():
                handle.release_memory()
