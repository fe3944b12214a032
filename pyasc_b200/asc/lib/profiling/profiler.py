from __future__ import annotations

import ctypes
import statistics
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Iterator, List, Optional

from .. import runtime as rt


@dataclass
class Task:
    name: str
    duration_us: float


@dataclass
class ProfilingResult:
    tasks: List[Task] = field(default_factory=list)


def task_time_median(tasks: List[Task], skip: int = 0) -> float:
    """Median task duration in microseconds, ignoring the first ``skip`` tasks (warm-up)."""
    durations = [t.duration_us for t in tasks[skip:]]
    if not durations:
        raise ValueError("No profiled tasks")
    return statistics.median(durations)


class Profiler:
    """``with profiler.profile(): kernel[...](...)`` records one task per region."""

    def __init__(self, output_dir: Optional[str] = None):
        self.output_dir = output_dir
        self.last_result = ProfilingResult()

    @staticmethod
    def _event() -> ctypes.c_void_p:
        ev = ctypes.c_void_p()
        rt.state.lib.call("asc_cuda_event_create", ctypes.c_void_p(ctypes.addressof(ev)))
        return ev

    @contextmanager
    def profile(self, name: str = "kernel") -> Iterator["Profiler"]:
        stream = rt.current_stream()
        start, stop = self._event(), self._event()
        call = rt.state.lib.call
        call("asc_cuda_event_record", start, stream)
        try:
            yield self
        finally:
            call("asc_cuda_event_record", stop, stream)
            call("asc_cuda_event_synchronize", stop)
            ms = ctypes.c_float(0)
            call("asc_cuda_event_elapsed_ms", start, stop, ctypes.c_void_p(ctypes.addressof(ms)))
            self.last_result.tasks.append(Task(name, ms.value * 1e3))
            call("asc_cuda_event_destroy", start)
            call("asc_cuda_event_destroy", stop)
