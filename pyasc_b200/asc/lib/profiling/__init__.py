"""Kernel timing for the CUDA platform (reference: python/asc/lib/profiling/: ``Profiler`` wraps
libmsprofiler and parses its CSV export, profiler.py:59-129; ``task_time_median``, result.py:33-47).
Here a profiled region is bracketed by CUDA events on the runtime's current stream."""
from .profiler import Profiler, ProfilingResult, task_time_median  # noqa: F401
