"""Kernels specialised at first use of an expression.

The generic elementwise and row-program kernels of libasc_cuda interpret a postfix program, which costs issue
slots.  The same machine exists with the opcode list as a template argument (``Compiled`` / ``RowStep`` in
``csrc/eltwise_program.cuh``): every dispatch folds away and the stack lives in registers.  This module turns any
program the launcher plans into such a kernel: it writes a translation unit of a few lines that instantiates the
executor for the program's opcode list, compiles it with nvcc into a small shared library, keeps the library in a
file cache keyed by the content hash of everything that went into it, loads it and registers its entry point with
libasc_cuda (``asc_cuda_register_program``).  From then on the library runs that kernel whenever the program is
submitted; until the build has finished, and where no compiler is installed, the interpreter runs it, with
bit-identical results (the arithmetic of both is the same ``apply_binary`` / ``apply_unary`` code).

This is the CUDA platform's counterpart of the reference's first-use compilation and its cache
(python/asc/runtime/jit.py:158-202, python/asc/runtime/cache.py:31-162, python/asc/lib/runtime/state.py:36-48):
``PYASC_CACHE_DIR`` names the cache directory there and here (default here: ``lib/jit`` inside the package, so that
libraries built on one machine travel with the tree).  ``ASC_CUDA_JIT`` = ``0`` switches the mechanism off,
``sync`` builds in the foreground (the first launch already runs the specialised kernel), anything else builds on
a background thread.
"""
from __future__ import annotations

import atexit
import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

from . import build as _build

OP_LOAD, OP_TEE, OP_TMP = 0, 63, 64
ROW_SCALAR_WORD = 1 << 24
ROW_KIND = 1000                      # kind of a row program with kV columns per thread: ROW_KIND + kV

Key = Tuple[int, Tuple[int, ...]]

_lock = threading.Lock()
_registered: Dict[Key, ctypes.CDLL] = {}       # loaded and registered (the CDLL object keeps the code mapped)
_pending: Dict[Key, bool] = {}                   # queued or being built
_queue: List[Key] = []
_workers = 0
_stopping = False
_failed: Dict[Key, str] = {}
_exit_hook = False
builds: List[str] = []                          # paths of the libraries built or loaded in this process


def mode() -> str:
    return os.environ.get("ASC_CUDA_JIT", "async").lower()


def cache_dir() -> Path:
    return Path(os.environ.get("PYASC_CACHE_DIR") or (_build.LIB_DIR / "jit"))


def program_words(ops: Sequence[int], args: Sequence[int], row_scalar_inputs: Sequence[bool] = ()) -> Tuple[int, ...]:
    """The words the generated unit's ``OpList`` holds: opcode (with the immediate flag), the input index of a LOAD or
    the slot of a TEE / TMP in bits 16-23, bit 24 on a LOAD of an input that holds one element per row."""
    words = []
    for op, arg in zip(ops, args):
        w = int(op)
        code = w & 0xff
        if code in (OP_LOAD, OP_TEE, OP_TMP):
            w |= int(arg) << 16
        if code == OP_LOAD and row_scalar_inputs and row_scalar_inputs[int(arg)]:
            w |= ROW_SCALAR_WORD
        words.append(w)
    return tuple(words)


def row_kind(cols: int) -> int:
    kv = 1
    while kv * 256 < cols:
        kv *= 2
    return ROW_KIND + kv


def _fingerprint() -> bytes:
    h = hashlib.blake2b(digest_size=16)
    for name in ("eltwise_program.cuh", "common.cuh"):
        h.update((_build.CSRC / name).read_bytes())
    h.update(" ".join(_build.NVCC_FLAGS).encode())
    return h.digest()


def library_name(kind: int, words: Sequence[int]) -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(_fingerprint())
    h.update(repr((kind, tuple(words))).encode())
    return f"prog_{h.hexdigest()}.so"


def source(kind: int, words: Sequence[int]) -> str:
    header = (_build.CSRC / "eltwise_program.cuh").as_posix()
    body = ", ".join(str(w) for w in words)
    if kind >= ROW_KIND:
        call = f"jit_launch_row<P, {kind - ROW_KIND}>(*static_cast<const EltProgram*>(prog), n, flag, sms, static_cast<cudaStream_t>(stream))"
    else:
        call = "jit_launch_eltwise<P>(*static_cast<const EltProgram*>(prog), n, flag, sms, static_cast<cudaStream_t>(stream))"
    return (f'#include "{header}"\n'
            f"namespace {{ using P = OpList<{body}>; }}\n"
            'extern "C" int asc_jit_run(const void* prog, long long n, int flag, int sms, void* stream) {\n'
            f"  return {call};\n"
            "}\n")


def compiler() -> Optional[str]:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else None


def build_library(kind: int, words: Sequence[int]) -> Path:
    """Compile (or find in the cache) the library for one program; returns its path."""
    out = cache_dir() / library_name(kind, words)
    if out.exists():
        return out
    nvcc = compiler()
    if nvcc is None:
        raise RuntimeError("nvcc not found: programs cannot be specialised, the interpreter runs them")
    out.parent.mkdir(parents=True, exist_ok=True)
    src = out.with_suffix(f".{os.getpid()}.{threading.get_ident()}.cu")
    tmp = out.with_suffix(f".{os.getpid()}.{threading.get_ident()}.tmp")
    src.write_text(source(kind, words))
    try:
        cmd = [nvcc, *_build.NVCC_FLAGS, "-shared", "-I", str(_build.INCLUDE), "-o", str(tmp), str(src)]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for a specialised program:\n{res.stdout}")
        os.replace(tmp, out)            # atomic: another process sees the whole file or none
    finally:
        for f in (src, tmp):
            try:
                f.unlink()
            except FileNotFoundError:
                pass
    return out


def _load_and_register(key: Key, path: Path) -> None:
    from . import capi
    kind, words = key
    lib = ctypes.CDLL(str(path))
    fn = ctypes.cast(lib.asc_jit_run, ctypes.c_void_p)
    arr = (ctypes.c_int32 * len(words))(*words)
    capi.call("asc_cuda_register_program", ctypes.c_int32(kind), arr, ctypes.c_int32(len(words)), fn)
    with _lock:
        _registered[key] = lib
        builds.append(str(path))


def _build_and_register(key: Key) -> None:
    try:
        _load_and_register(key, build_library(*key))
    except Exception as e:          # a failed build leaves the interpreter in charge; the reason is kept
        with _lock:
            _failed[key] = str(e)
    finally:
        with _lock:
            _pending.pop(key, None)


MAX_BUILDERS = 2        # nvcc processes this module runs at a time


def _worker() -> None:
    while True:
        with _lock:
            if _stopping or not _queue:
                global _workers
                _workers -= 1
                return
            key = _queue.pop(0)
        _build_and_register(key)


def min_elements() -> int:
    """Launches that touch fewer elements than this keep the interpreter: the build would cost more than it saves."""
    return int(os.environ.get("ASC_CUDA_JIT_MIN_ELEMENTS", str(1 << 15)))


def request(kind: int, words: Sequence[int], wait: bool = False) -> bool:
    """Make sure the specialised kernel for this program exists or is being built.  Returns True when it is
    registered (the next launch runs it), False while the interpreter still serves the program."""
    global _workers, _exit_hook
    if mode() in ("0", "off", "no", "false") or not words:
        return False
    key: Key = (int(kind), tuple(int(w) for w in words))
    with _lock:
        if key in _registered:
            return True
        if key in _failed:
            return False
        queued = key in _pending
    if not queued:
        cached = cache_dir() / library_name(*key)
        if cached.exists() or wait or mode() == "sync":
            _build_and_register(key)
            return key in _registered
        with _lock:
            if key not in _pending:
                _pending[key] = True
                _queue.append(key)
                if _workers < MAX_BUILDERS:
                    _workers += 1
                    threading.Thread(target=_worker, daemon=True).start()
                if not _exit_hook:
                    atexit.register(_shutdown)
                    _exit_hook = True
    if wait or mode() == "sync":     # also when another caller queued this program before: its build is under way
        wait_all()
    return key in _registered


def prepare(plan, wait: bool = False) -> int:
    """Requests the specialised kernel of every program step of a launch plan that is large enough to gain from it;
    returns how many are registered."""
    ready = 0
    work: Dict[Key, int] = {}
    for step in plan.steps:
        prog = getattr(step, "program", None)
        if prog is not None:
            work[prog] = work.get(prog, 0) + int(getattr(step, "elements", 0))
    least = 0 if wait else min_elements()
    for prog, elements in work.items():
        if elements >= least and request(prog[0], prog[1], wait=wait):
            ready += 1
    return ready


def wait_all() -> None:
    """Blocks until every build requested so far has finished."""
    import time
    while True:
        with _lock:
            if not _pending:
                return
        time.sleep(0.02)


def _shutdown() -> None:
    """At interpreter exit: builds not yet started are dropped, the ones running finish (their libraries land in
    the cache whole)."""
    global _stopping
    import time
    with _lock:
        _stopping = True
        for key in _queue:
            _pending.pop(key, None)
        _queue.clear()
    deadline = time.time() + 30
    while time.time() < deadline:
        with _lock:
            if not _pending:
                return
        time.sleep(0.02)


def failures() -> Dict[Key, str]:
    with _lock:
        return dict(_failed)
