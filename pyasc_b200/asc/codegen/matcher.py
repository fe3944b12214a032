"""Maps a recorded kernel onto the hand-written CUDA kernels of libasc_cuda.

The reference lowers the recorded tile ops through ``asctile`` -> ``ascendc`` -> Ascend C and runs
``core_num`` blocks (lib/Conversion/LowerToAsc/*.cpp).  The CUDA platform instead recognises the
whole-kernel pattern and launches one fused CUDA kernel that produces the same result over the part
of each tensor the blocks would have touched together.  For that it

1. evaluates every load/store offset for all blocks and loop iterations at once (NumPy), honouring
   the reference's boundary rules: loads past the tensor end are padded, stores are clipped
   (LowerAscTileDataTransfer.cpp:184-218, 254-261);
2. checks that the touched tiles form contiguous ranges / full tile grids and merges them;
3. emits :class:`Step` objects, each one C-ABI call with concrete sizes and byte offsets.

A kernel that fits no pattern raises ``NotImplementedError``: there is no host-side interpreter, Triton or CPU
fallback behind this module.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..language.core.dtype import DataType, KnownTypes as KT
from ..language.core.ir_value import PlainValue, same_scalar
from ..language.tile.tensor import Tensor
from ..language.tile.tile import Tile
from ..language.tile.trace import Effect, Loop, Node
from .tracer import KernelTrace

MAX_INSTANCES = 1 << 26     # (block, iteration) combinations the matcher is willing to enumerate
MAX_CALLS = 4096            # C-ABI calls one kernel launch may expand to

_DTYPE_CODE_16 = {"float16": 0, "bfloat16": 1}
_OUT_CODE = {"float16": 0, "bfloat16": 1, "float32": 2}


class UnsupportedKernelError(NotImplementedError):
    pass


def _unsupported(msg: str) -> UnsupportedKernelError:
    return UnsupportedKernelError(f"The CUDA platform has no kernel for this pattern: {msg}")


# --------------------------------------------------------------------------------------------------
# Plan
# --------------------------------------------------------------------------------------------------
class Step:
    """One C-ABI call.  ``build(ptrs, stream)`` returns the ctypes argument list; ``ptrs`` maps a
    runtime-argument index (or a temp-buffer key) to a device address."""

    def __init__(self, fn_name: str, build: Callable[[Dict[Any, int], Any], Sequence[Any]], note: str = ""):
        self.fn_name = fn_name
        self.build = build
        self.note = note
        self.program = None      # (kind, opcode-list words) of an elementwise / row program step, see pyasc_b200/jit.py
        self.elements = 0        # elements such a step computes

    def __repr__(self) -> str:
        return f"Step({self.fn_name}: {self.note})"


class PipelineSpec:
    """How a one-call plan that overwrites its outputs completely splits into independent chunks along
    its unit axis (elements, softmax rows, GEMM rows of A and C, attention heads), so that the launcher
    can overlap the upload of chunk i+1, the kernel of chunk i and the download of chunk i-1."""

    def __init__(self, units: int, granule: int, streamed: Dict[int, int], resident: set,
                 make_steps: Callable[[int, int], List["Step"]]):
        self.units = units            # length of the unit axis
        self.granule = granule        # chunk boundaries are multiples of this many units
        self.streamed = streamed      # argument index -> bytes per unit (argument is sliced along the axis)
        self.resident = resident      # argument indices every chunk needs whole (uploaded first)
        self.make_steps = make_steps  # C-ABI calls for units [lo, hi)


class Plan:

    def __init__(self, pattern: str):
        self.pattern = pattern
        self.steps: List[Step] = []
        self.reads: set = set()       # runtime-argument indices the kernel reads
        self.writes: set = set()      # ... and writes
        self.partial_writes: set = set()  # written arguments whose buffer is not overwritten completely
        self.temps: Dict[str, int] = {}  # temp-buffer key -> bytes
        self.pipeline: Optional[PipelineSpec] = None

    def __repr__(self) -> str:
        return f"Plan({self.pattern}, steps={self.steps}, reads={sorted(self.reads)}, writes={sorted(self.writes)})"


def _p(addr: int) -> ctypes.c_void_p:
    return ctypes.c_void_p(addr)


# --------------------------------------------------------------------------------------------------
# Enumerating (block, iteration) instances of a loop nest
# --------------------------------------------------------------------------------------------------
def enumerate_instances(core_num: int, loops: Tuple[Loop, ...], guards: Tuple = ()) -> Dict[str, np.ndarray]:
    """Symbol bindings, one array entry per (block, iteration...) combination of ``loops`` for which every guard
    (an ``if`` condition on the block index or a loop variable, with the outcome the effect lies under) holds."""
    if guards:
        env = enumerate_instances(core_num, loops)
        n = env_count(env)
        keep = np.ones(n, dtype=bool)
        for cond, outcome in guards:
            try:
                value = np.broadcast_to(np.asarray(cond.evaluate(env)), (n, )) != 0
            except Exception as e:
                raise _unsupported("'if' on a scalar that is not a function of the block index, loop variables and "
                                   f"launch arguments ({e})") from None
            keep &= value if outcome else ~value
        return {name: arr[keep] for name, arr in env.items()}
    env: Dict[str, np.ndarray] = {"block_idx": np.arange(core_num, dtype=np.int64)}
    count = core_num
    for loop in loops:
        start = np.broadcast_to(np.asarray(loop.start.evaluate(env), dtype=np.int64), (count, ))
        stop = np.broadcast_to(np.asarray(loop.stop.evaluate(env), dtype=np.int64), (count, ))
        step = np.broadcast_to(np.asarray(loop.step.evaluate(env), dtype=np.int64), (count, ))
        if np.any(step <= 0):
            raise _unsupported("loop with a non-positive step")
        trips = np.maximum(0, -((start - stop) // step))
        total = int(trips.sum())
        if total > MAX_INSTANCES:
            raise _unsupported(f"loop nest expands to {total} iterations; use larger tiles")
        rep = np.repeat(np.arange(count), trips)
        first = np.cumsum(trips) - trips
        k = np.arange(total, dtype=np.int64) - np.repeat(first, trips)
        env = {name: arr[rep] for name, arr in env.items()}
        env[loop.name] = start[rep] + k * step[rep]
        count = total
    return env


def eval_int(value: PlainValue, env: Dict[str, np.ndarray], count: int) -> np.ndarray:
    return np.broadcast_to(np.asarray(value.evaluate(env), dtype=np.int64), (count, )).copy()


def env_count(env: Dict[str, np.ndarray]) -> int:
    return int(next(iter(env.values())).shape[0])


def merge_intervals(starts: np.ndarray, ends: np.ndarray) -> List[Tuple[int, int]]:
    """Union of half-open intervals as a sorted list of disjoint ones."""
    keep = ends > starts
    starts, ends = starts[keep], ends[keep]
    if starts.size == 0:
        return []
    order = np.argsort(starts, kind="stable")
    starts, ends = starts[order], ends[order]
    run_max = np.maximum.accumulate(ends)
    breaks = np.nonzero(starts[1:] > run_max[:-1])[0] + 1
    firsts = np.concatenate(([0], breaks))
    lasts = np.concatenate((breaks, [starts.size])) - 1
    return [(int(starts[f]), int(run_max[l])) for f, l in zip(firsts, lasts)]


# --------------------------------------------------------------------------------------------------
# Views of global tensors
# --------------------------------------------------------------------------------------------------
class GmView:
    """A tile that is (a sub-window of) a load from a global tensor."""

    def __init__(self, tensor: Tensor, offsets: Tuple[PlainValue, ...], shape: Tuple[int, ...], pad_value: Any = 0):
        self.tensor = tensor
        self.offsets = offsets
        self.shape = shape
        self.pad_value = pad_value


def resolve_view(tile: Any) -> Optional[GmView]:
    if not isinstance(tile, Tile):
        return None
    node = tile.node
    if id(node) in _MATERIALISED:           # a value already planned into a temporary reads like a load from it
        op = _MATERIALISED[id(node)]
        if op.bcast or op.scalar or op.per_row:
            return None
        return GmView(op.tensor, op.offsets, op.shape, 0)
    if node.kind == "load":
        return GmView(node.args[0], node.attrs["offsets"], node.attrs["shape"], node.attrs["pad_value"])
    if node.kind == "copy":
        inner = resolve_view(node.args[0])
        if inner is None:
            return None
        offs = tuple(a + b for a, b in zip(inner.offsets, node.attrs["offsets"]))
        return GmView(inner.tensor, offs, node.attrs["shape"], inner.pad_value)
    return None


def _is_materialised(tile: Any) -> bool:
    return isinstance(tile, Tile) and id(tile.node) in _MATERIALISED


def _is_zero_pad(view: GmView) -> bool:
    pv = view.pad_value
    if isinstance(pv, PlainValue):
        return pv.is_const and pv.value == 0
    return pv == 0 or pv is None


def _row_major_2d(t: Tensor) -> Tuple[int, int]:
    shape = t.static_shape()
    if len(shape) == 1:
        return 1, shape[0]
    if len(shape) == 2:
        return shape
    raise _unsupported(f"tensor of rank {len(shape)}")


def _check_fits(t: Tensor) -> None:
    n = 1
    for d in t.static_shape():
        n *= d
    if n > t.base.numel:
        raise RuntimeError(f"asc2.tensor({t.base.name}, {list(t.static_shape())}) describes {n} elements but the "
                           f"argument holds {t.base.numel}")


# --------------------------------------------------------------------------------------------------
# Small structural helpers
# --------------------------------------------------------------------------------------------------
def _node(tile: Any, _kind: str, /, **attrs) -> Optional[Node]:
    """The tile's defining node if it is of ``kind`` with the given attribute values."""
    if not isinstance(tile, Tile) or tile.node.kind != _kind:
        return None
    for k, v in attrs.items():
        if tile.node.attrs.get(k) != v:
            return None
    return tile.node


def _tile_scalar_node(value: Any, _kind: str, /, **attrs) -> Optional[Node]:
    """``value`` is the scalar result of a no-axis reduction (or scalar load) node of ``kind``."""
    if not isinstance(value, PlainValue) or value.op != "tile_scalar":
        return None
    node = value.args[0]
    if node.kind != _kind:
        return None
    for k, v in attrs.items():
        if node.attrs.get(k) != v:
            return None
    return node


def _same_offsets(a: Sequence[PlainValue], b: Sequence[PlainValue]) -> bool:
    return len(a) == len(b) and all(same_scalar(x, y) for x, y in zip(a, b))


def _flat_window(view_tensor: Tensor, offsets: Sequence[PlainValue], shape: Tuple[int, ...]):
    """For a tile that covers whole rows of a row-major tensor (or any 1-D tile): returns
    ``(flat_offset_expr, elements)``; ``None`` when the tile is not one contiguous range."""
    tshape = view_tensor.static_shape()
    if len(tshape) != len(shape):
        return None
    if len(shape) == 1:
        return offsets[0], shape[0]
    # all trailing dims must span the tensor fully and start at 0
    for d in range(1, len(shape)):
        if shape[d] != tshape[d] or not (offsets[d].is_const and offsets[d].value == 0):
            return None
    inner = 1
    for d in tshape[1:]:
        inner *= d
    return offsets[0] * inner, shape[0] * inner


# --------------------------------------------------------------------------------------------------
# Pattern: elementwise map over same-offset loads (x + y, x * y + z)
# --------------------------------------------------------------------------------------------------
def _match_elementwise(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    value, out_t = eff.args
    offsets = eff.attrs["offsets"]
    if not isinstance(value, Tile):
        return None

    def leaf(tile: Any) -> Optional[GmView]:
        v = resolve_view(tile) if _node(tile, "load") else None
        if v is None or v.shape != value.shape or not _same_offsets(v.offsets, offsets):
            return None
        if v.tensor.static_shape() != out_t.static_shape():
            return None
        return v

    top = _node(value, "binary", op="add")
    if top is None:
        return None
    lhs, rhs = top.args
    operands: List[GmView] = []
    fn_name = None
    if leaf(lhs) is not None and leaf(rhs) is not None:
        operands = [leaf(lhs), leaf(rhs)]
        fn_name = "asc_cuda_vadd_f32"
    else:
        for prod, addend in ((lhs, rhs), (rhs, lhs)):
            m = _node(prod, "binary", op="mul")
            if m is not None and leaf(m.args[0]) is not None and leaf(m.args[1]) is not None \
                    and leaf(addend) is not None:
                operands = [leaf(m.args[0]), leaf(m.args[1]), leaf(addend)]
                fn_name = "asc_cuda_vmuladd_f32"
                break
    if fn_name is None:
        return None
    if value.dtype != KT.float32 or out_t.dtype != KT.float32 or any(v.tensor.dtype != KT.float32 for v in operands):
        return None  # the generic elementwise program handles the other types
    window = _flat_window(out_t, offsets, value.shape) if eff.kind == "store" else None
    if window is None:
        return None   # 2-D tiles that do not span whole rows: the program kernel handles windows
    _check_fits(out_t)
    for v in operands:
        _check_fits(v.tensor)
    flat_off, tile_elems = window
    numel = 1
    for d in out_t.static_shape():
        numel *= d
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    starts = eval_int(flat_off, env, n)
    if starts.size and starts.min() < 0:
        raise RuntimeError("Negative tile offset in kernel")
    ends = np.minimum(starts + tile_elems, numel)
    intervals = merge_intervals(starts, ends)
    if len(intervals) > MAX_CALLS:
        raise _unsupported("elementwise kernel touching more than 4096 disjoint ranges")

    plan = Plan("elementwise:" + fn_name)
    out_idx = out_t.base.index
    in_idx = [v.tensor.base.index for v in operands]
    plan.reads.update(in_idx)
    plan.writes.add(out_idx)
    if intervals != [(0, out_t.base.numel)]:
        plan.partial_writes.add(out_idx)
    def make(lo: int, hi: int) -> List[Step]:
        def build(ptrs, stream, lo=lo, hi=hi):
            args = [_p(ptrs[i] + 4 * lo) for i in in_idx]
            return (*args, _p(ptrs[out_idx] + 4 * lo), ctypes.c_int64(hi - lo), stream)
        return [Step(fn_name, build, f"[{lo}, {hi})")]

    for lo, hi in intervals:
        plan.steps += make(lo, hi)
    if not plan.partial_writes and len(intervals) == 1:
        plan.pipeline = PipelineSpec(intervals[0][1], 1 << 16, {i: 4 for i in in_idx + [out_idx]}, set(), make)
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: any elementwise expression over same-offset loads -> one postfix program, one pass
# --------------------------------------------------------------------------------------------------
_OP_LOAD, _OP_CONST, _OP_WHERE, _OP_ROUND_F16, _OP_ROUND_BF16 = 0, 1, 32, 33, 34
_BINARY_CODE = {"add": 2, "sub": 3, "mul": 4, "div": 5, "max": 6, "min": 7}
_UNARY_CODE = {"neg": 8, "abs": 9, "relu": 10, "exp": 11, "exp2": 12, "log": 13, "log2": 14, "sqrt": 15, "rsqrt": 16,
               "sin": 17, "cos": 18, "tan": 19, "sinh": 20, "cosh": 21, "tanh": 22, "erf": 23, "floor": 24, "ceil": 25}
_COMPARE_CODE = {"eq": 26, "ne": 27, "gt": 28, "ge": 29, "lt": 30, "le": 31}
_INT_BINARY_CODE = {"add": 35, "sub": 36, "mul": 37, "max": 38, "min": 39, "shl": 40, "shr": 41}
_INT_COMPARE_CODE = {"eq": 42, "ne": 43, "gt": 44, "ge": 45, "lt": 46, "le": 47}
_INT_UNARY_CODE = {"neg": 48, "abs": 49, "relu": 50}
_OP_CVT_I2F, _OP_CVT_F2I, _OP_WRAP_I16 = 51, 52, 53
_ELT_TYPE = {"float32": 0, "float16": 1, "bfloat16": 2, "int32": 3, "int16": 4}
# 8-bit integers are storage types: a program may load them (to compare, or to cast to a wider integer) and may
# store an int32 cast to them; it does not compute on 8-bit tiles (that would need a wrap after every operation).
# The kernels never see them: an int8 / uint8 tensor a program loads is first widened, whole, into an int32
# temporary (its "twin"), and an 8-bit result is narrowed out of one (asc_cuda_convert_bytes).
_BYTE_TYPES = ("int8", "uint8")
_STORAGE_TYPE = frozenset(_ELT_TYPE) | frozenset(_BYTE_TYPES)      # element types a program may load or compare
_ROUND_CODE = {"float16": _OP_ROUND_F16, "bfloat16": _OP_ROUND_BF16, "int16": _OP_WRAP_I16}
ELT_MAX_OPS, ELT_MAX_INPUTS, ELT_MAX_STACK = 48, 6, 8
_ROW_CODE = {"sum": 59, "max": 60, "min": 61, "prod": 62}     # row programs: reduce the top of the stack over the row
ROW_MAX_COLS = 8192
ROW_MAX_TMP = 4
_ROW_SCALAR_INPUT = 0x200    # flag on an input type: one element per row (address = row * pitch)
_OP_TEE, _OP_TMP = 63, 64     # row programs: copy the top into / push temporary slot arg
_OP_INDEX = 65                # push the element's row-major index inside the call's window (int32)
_MARK_BEGIN, _MARK_END = -1, -2   # pseudo-ops around the code of one traced value (arg: its identity)


def _round_const(value: float, dtype: DataType) -> float:
    """A scalar operand takes the tile's type (python/asc/language/tile/utils.py:73-94)."""
    if dtype.name == "float16":
        return float(np.float16(value))
    if dtype.name == "bfloat16":
        bits = np.array([value], dtype=np.float32).view(np.uint32).astype(np.uint64)
        bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16  # round to nearest even
        return float(bits.astype(np.uint32).view(np.float32)[0])
    return float(np.float32(value))


_OP_IMM = 0x100
# opcode whose operands are swapped: _SWAPPED[op](b, a) == op(a, b)
_SWAPPED = {2: 2, 4: 4, 6: 6, 7: 7, 3: 54, 5: 55, 26: 26, 27: 27, 28: 30, 30: 28, 29: 31, 31: 29,
            35: 35, 37: 37, 38: 38, 39: 39, 36: 56, 40: 57, 41: 58, 42: 42, 43: 43, 44: 46, 46: 44, 45: 47, 47: 45}


class _Frag:
    """Postfix code that leaves one value on the stack; ``need`` is the stack depth it uses.  A
    constant is kept as its 32-bit word until its consumer decides between an immediate operand and a
    CONST push."""

    __slots__ = ("code", "need", "word")

    def __init__(self, code: List[Tuple[int, int]], need: int, word: Optional[int] = None):
        self.code, self.need, self.word = code, need, word

    def pushed(self) -> "_Frag":
        return _Frag([(_OP_CONST, self.word)], 1) if self.word is not None else self


class _Operand:
    """One LOAD source of a program: the tile of ``shape`` loaded from ``tensor`` at ``offsets``.  ``bcast``: the
    tile is a single row that every row of the result repeats; ``scalar``: one element (a scalar load)."""

    __slots__ = ("tensor", "offsets", "shape", "bcast", "scalar", "per_row")

    def __init__(self, tensor: Tensor, offsets: Sequence[PlainValue], shape: Tuple[int, ...], bcast: bool = False,
                 scalar: bool = False, per_row: bool = False):
        self.tensor, self.offsets, self.shape, self.bcast, self.scalar = tensor, tuple(offsets), tuple(shape), bcast, scalar
        self.per_row = per_row      # one element per row of the result, repeated along the row (row programs)

    def same(self, o: "_Operand") -> bool:
        return (self.tensor.base.index == o.tensor.base.index and self.tensor.dtype == o.tensor.dtype
                and self.tensor.static_shape() == o.tensor.static_shape() and self.shape == o.shape
                and self.bcast == o.bcast and self.scalar == o.scalar and self.per_row == o.per_row
                and _same_offsets(self.offsets, o.offsets))

    def addressed_like(self, out_t: Tensor, offsets: Sequence[PlainValue], shape: Tuple[int, ...]) -> bool:
        """Same tile of a same-shaped tensor as the store: element i of the operand is element i of the result."""
        return (not self.bcast and self.tensor.static_shape() == out_t.static_shape() and self.shape == tuple(shape)
                and _same_offsets(self.offsets, offsets))


# Values that are read back from a temporary device buffer instead of being compiled into the program: node id ->
# the operand to load.  Filled only while _match_matmul_then_program and _match_column_statistics plan the expression
# around a value they have already planned into a temporary (a matmul result, a reduction along the first axis).
class _Materialised(threading.local):
    """Per thread, so that kernels planned from different threads do not see each other's temporaries."""

    def __init__(self):
        self.table: Dict[int, "_Operand"] = {}

    def __contains__(self, key: int) -> bool:
        return key in self.table

    def __getitem__(self, key: int) -> "_Operand":
        return self.table[key]

    def __setitem__(self, key: int, value: "_Operand") -> None:
        self.table[key] = value

    def __bool__(self) -> bool:
        return bool(self.table)

    def clear(self) -> None:
        self.table.clear()


_MATERIALISED = _Materialised()


class _EltProgram:
    """Compiles the expression tree of a stored tile into a postfix program.  Scalar operands become
    immediates; of two tile operands the one needing the deeper stack is evaluated first (with the
    swapped opcode when that reverses the order), which keeps most expressions at depth 2."""

    def __init__(self, shape, offsets, out_t: Tensor, scalar_store: bool = False):
        self.shape, self.offsets, self.out_t = tuple(shape), offsets, out_t
        self.scalar_store = scalar_store
        self.operands: List[_Operand] = []
        self.reshaped = False       # a reshape was seen: element order is the flat (row-major) order
        self.row_ops = False        # the program reduces over rows: it runs as a row program
        self.uses_index = False     # the program reads the element index inside the tile: one call per tile
        self.row_expr = False       # generating code for a [1, cols] row that every row of the result repeats
        self.whole_tile = False     # a reduction of a whole multi-row tile: the tile is walked as one long row
        self.per_row_reductions = False
        self.n_tmp = 0              # temporary slots the finished program uses
        self.visits = 0             # values visited while generating code
        self.root: Any = None       # the value compile() was asked for (the one the program stores)
        self.expanded: Dict[int, Tile] = {}   # asc2.softmax nodes of computed tiles -> their row-reduction expression
        self.allow_bytes = False    # the caller widens int8 / uint8 operands into int32 twins before the program runs
        self.twins: Dict[str, Tuple[Tensor, Tensor]] = {}   # twin key -> (int32 twin, the 8-bit tensor)
        self.full_shape: Optional[Tuple[int, ...]] = None   # set while code for a per-row value is generated
        self.ops: List[int] = []
        self.args: List[int] = []
        self.max_depth = 0

    @property
    def inputs(self) -> List[Tensor]:
        return [o.tensor for o in self.operands]

    @staticmethod
    def _word(value: Any, dtype: DataType) -> int:
        """``value`` as a scalar of ``dtype``: a scalar operand takes the tile's type."""
        if dtype.is_float():
            return int(np.array([_round_const(float(value), dtype)], dtype=np.float32).view(np.int32)[0])
        if float(value) != int(value):
            raise _unsupported(f"scalar {value} combined with a tile of {dtype}")
        wrapped = np.array([int(value)], dtype=np.int64).astype(np.int16 if dtype.name == "int16" else np.int32)
        return int(wrapped[0])

    @staticmethod
    def _rounded(frag: _Frag, dtype: DataType) -> _Frag:
        if dtype.name in _ROUND_CODE:
            return _Frag(frag.code + [(_ROUND_CODE[dtype.name], 0)], frag.need)
        return frag

    def _binary(self, code: int, lhs: _Frag, rhs: _Frag) -> _Frag:
        if rhs.word is not None and lhs.word is None:
            return _Frag(lhs.code + [(_SWAPPED[code] | _OP_IMM, rhs.word)], lhs.need)
        if lhs.word is not None and rhs.word is None:
            return _Frag(rhs.code + [(code | _OP_IMM, lhs.word)], rhs.need)
        lhs, rhs = lhs.pushed(), rhs.pushed()
        if rhs.need > lhs.need:
            return _Frag(rhs.code + lhs.code + [(_SWAPPED[code], 0)], max(rhs.need, lhs.need + 1))
        return _Frag(lhs.code + rhs.code + [(code, 0)], max(lhs.need, rhs.need + 1))

    def _twin(self, tensor: Tensor) -> Tensor:
        """The int32 stand-in of an int8 / uint8 tensor (one per tensor, so that equal operands stay equal)."""
        key = _twin_key(tensor)
        if key not in self.twins:
            self.twins[key] = (_fake_like(key, tensor, KT.int32), tensor)
        return self.twins[key][0]

    def _load(self, operand: _Operand) -> Optional[_Frag]:
        if operand.tensor.dtype.name in _BYTE_TYPES:
            if not self.allow_bytes:
                return None
            operand = _Operand(self._twin(operand.tensor), operand.offsets, operand.shape, operand.bcast, operand.scalar,
                               operand.per_row)
        if operand.tensor.dtype.name not in _ELT_TYPE:
            return None
        for k, o in enumerate(self.operands):
            if o.same(operand):
                return _Frag([(_OP_LOAD, k)], 1)
        self.operands.append(operand)
        return _Frag([(_OP_LOAD, len(self.operands) - 1)], 1)

    def _view_operand(self, tile: Tile, bcast: bool = False) -> Optional[_Frag]:
        view = resolve_view(tile) if tile.node.kind in ("load", "copy") else None
        if view is None or not _is_zero_pad(view):
            return None
        return self._load(_Operand(view.tensor, view.offsets, view.shape, bcast))

    def gen(self, v: Any, scalar_dtype: Optional[DataType] = None) -> Optional[_Frag]:
        """Code for ``v``, or None when ``v`` is not expressible.  The code of every traced value is bracketed by
        markers that name the value, so that ``_finish`` can see which values an expression uses more than once."""
        self.visits += 1
        if self.visits > 8 * ELT_MAX_OPS * ELT_MAX_OPS:
            # an expression graph that shares subexpressions unfolds into a tree here; one that unfolds into far
            # more nodes than a program may hold is refused before the unfolding takes exponential time
            raise _unsupported(f"elementwise expression that unfolds into more than {self.visits - 1} operations")
        frag = self._gen(v, scalar_dtype)
        if frag is None or frag.word is not None or len(frag.code) < 2:
            return frag
        if isinstance(v, Tile):
            key = id(v.node)
        elif isinstance(v, PlainValue) and not v.is_const:
            key = id(v.args[0]) if v.op == "tile_scalar" else id(v)
        else:
            return frag
        return _Frag([(_MARK_BEGIN, key)] + frag.code + [(_MARK_END, key)], frag.need)

    def _gen(self, v: Any, scalar_dtype: Optional[DataType] = None) -> Optional[_Frag]:
        if isinstance(v, PlainValue):
            if v.is_const:
                return _Frag([], 0, self._word(v.value, scalar_dtype or v.dtype))
            if v.op == "tile_scalar" and v.args[0].kind == "reduce" and not self.scalar_store:
                # the reduction of a whole one-row tile: a row reduction whose value every element sees
                return self._row_reduction(v.args[0], v.dtype)
            if v.op in ("sym", "tile_scalar") and not self.scalar_store:
                return None
            # a one-element store: scalars loaded from the stored position and arithmetic on them
            if v.op == "tile_scalar":
                node = v.args[0]
                if node.kind != "load_scalar":
                    return None
                return self._load(_Operand(node.args[0], node.attrs["offsets"], (1, ), scalar=True))
            code = (_BINARY_CODE if v.dtype.is_float() else _INT_BINARY_CODE).get(v.op)
            if code is None or v.dtype.name not in _ELT_TYPE or len(v.args) != 2:
                return None
            lhs, rhs = self.gen(v.args[0], v.dtype), self.gen(v.args[1], v.dtype)
            if lhs is None or rhs is None:
                return None
            return self._rounded(self._binary(code, lhs, rhs), v.dtype)
        if isinstance(v, (bool, int, float)):
            return _Frag([], 0, self._word(v, scalar_dtype or (KT.float32 if isinstance(v, float) else KT.int32)))
        if not isinstance(v, Tile):
            return None
        node = v.node
        if node.kind == "full":
            return self.gen(node.attrs["value"], v.dtype)
        if node.kind == "reduce" and self.full_shape is not None:
            return self._row_reduction(node, v.dtype)
        if v.shape != self.shape:
            return None
        if id(node) in _MATERIALISED:       # a value another kernel has written to a temporary (a matmul result)
            return self._load(_MATERIALISED[id(node)])
        if node.kind == "iota":
            if self.full_shape is not None:
                return None
            self.uses_index = True
            return _Frag([(_OP_INDEX, 0)], 1)
        if node.kind in ("load", "copy"):
            if self.full_shape is not None:
                # a loaded column: one element per row of the result; only a row program can address it
                view = resolve_view(v)
                if view is None or not _is_zero_pad(view):
                    return None
                self.row_ops = True
                return self._load(_Operand(view.tensor, view.offsets, view.shape, per_row=True))
            return self._view_operand(v, bcast=self.row_expr)
        if node.kind == "reshape":
            # row-major element order is kept, so elementwise code commutes with the reshape
            src = node.args[0]
            outer, self.shape = self.shape, src.shape
            try:
                frag = self.gen(src, scalar_dtype)
            finally:
                self.shape = outer
            if self.full_shape is None:
                self.reshaped = True      # (a per-row value has one element per row whatever its shape)
            return frag
        if node.kind == "broadcast":
            src = node.args[0]
            if _node(src, "full") is not None:
                return self.gen(src.node.attrs["value"], v.dtype)
            # a single row repeated along the leading dimension (also a loaded vector reshaped to one row)
            row = src
            while row.node.kind == "reshape" and row.node.args[0].size == row.size:
                row = row.node.args[0]
            if len(self.shape) == 2 and row.size == self.shape[1] and row.shape[-1] == self.shape[1] \
                    and src.shape[-1] == self.shape[1] and row.node.kind in ("load", "copy"):
                return self._view_operand(row, bcast=True)
            # a row computed from other rows (statistics along the first axis that have been written to a temporary, a
            # loaded row): every element evaluates the expression for its own column
            if len(self.shape) == 2 and self.full_shape is None and not self.row_expr and row.shape[-1] == self.shape[1] \
                    and row.size == self.shape[1] and _MATERIALISED:
                outer, self.shape, self.row_expr = self.shape, row.shape, True
                try:
                    return self.gen(row, scalar_dtype)
                finally:
                    self.shape, self.row_expr = outer, False
            # one value per row repeated along the row: an expression over reductions of tiles of this shape
            # along their last dimension (every element of the row evaluates it, the values agree)
            if len(self.shape) == 2 and self.full_shape is None and src.size == self.shape[0] \
                    and src.shape in ((self.shape[0], ), (self.shape[0], 1)):
                return self._per_row(src, self.shape)
            return None
        if node.kind == "softmax" and v.dtype == KT.float32 and len(v.shape) == 2:
            return self.gen(self._softmax_expression(v))
        if v.dtype.name not in _ELT_TYPE and node.kind != "compare":
            return None
        if node.kind == "binary":
            code = (_BINARY_CODE if v.dtype.is_float() else _INT_BINARY_CODE).get(node.attrs["op"])
            lhs, rhs = self.gen(node.args[0], v.dtype), self.gen(node.args[1], v.dtype)
            if code is None or lhs is None or rhs is None:
                return None
            return self._rounded(self._binary(code, lhs, rhs), v.dtype)
        if node.kind == "compare":
            dt = node.args[0].dtype
            if dt.name not in _STORAGE_TYPE:
                return None
            lhs, rhs = self.gen(node.args[0], dt), self.gen(node.args[1], dt)
            if lhs is None or rhs is None:
                return None
            return self._binary((_COMPARE_CODE if dt.is_float() else _INT_COMPARE_CODE)[node.attrs["mode"]], lhs, rhs)
        if node.kind == "where":
            parts = [self.gen(node.args[0]), self.gen(node.args[1], v.dtype), self.gen(node.args[2], v.dtype)]
            if any(p is None for p in parts) or parts[0].word is not None:
                return None
            c, a, b = (p.pushed() for p in parts)
            return _Frag(c.code + a.code + b.code + [(_OP_WHERE, 0)], max(c.need, a.need + 1, b.need + 2))
        if node.kind == "unary":
            code = (_UNARY_CODE if v.dtype.is_float() else _INT_UNARY_CODE).get(node.attrs["op"])
            src = self.gen(node.args[0])
            if code is None or src is None:
                return None
            src = src.pushed()
            return self._rounded(_Frag(src.code + [(code, 0)], src.need), v.dtype)
        if node.kind == "cast":
            src_t = node.args[0]
            src = self.gen(src_t) if src_t.dtype.name in _STORAGE_TYPE else None
            if src is None:
                return None
            src = src.pushed()
            if src_t.dtype.is_float() != v.dtype.is_float():
                src = _Frag(src.code + [(_OP_CVT_F2I if src_t.dtype.is_float() else _OP_CVT_I2F, 0)], src.need)
            return self._rounded(src, v.dtype)
        return None

    def _softmax_expression(self, v: Tile) -> Tile:
        """``asc2.softmax`` of a computed fp32 tile, spelled out as the row reductions a row program runs:
        ``e / sum(e)`` with ``e = exp(x - max(x))`` along the last dimension (python/asc/language/tile/unary_ops.py:213-223)."""
        cached = self.expanded.get(id(v.node))
        if cached is not None:
            return cached
        x, loops = v.node.args[0], v.node.loops
        last = len(x.shape) - 1
        column = x.shape[:-1] + (1, )

        def tile(of_shape, node_kind, args, attrs):
            return Tile(of_shape, x.dtype, Node(node_kind, args, attrs, loops), v.location)

        def along_rows(t, which):
            r = tile(column, "reduce", (t, ), {"kind": which, "dims": (last, ), "keep_dims": True})
            return tile(x.shape, "broadcast", (r, ), {"shape": x.shape})
        shifted = tile(x.shape, "binary", (x, along_rows(x, "max")), {"op": "sub"})
        e = tile(x.shape, "unary", (shifted, ), {"op": "exp"})
        out = tile(x.shape, "binary", (e, along_rows(e, "sum")), {"op": "div"})
        self.expanded[id(v.node)] = out
        return out

    def _per_row(self, v: Tile, full_shape: Tuple[int, ...]) -> Optional[_Frag]:
        """Code for a tile that holds one value per row of ``full_shape``."""
        outer, self.shape, self.full_shape = self.shape, v.shape, tuple(full_shape)
        try:
            return self.gen(v)
        finally:
            self.shape, self.full_shape = outer, None

    def _row_reduction(self, node: Node, dtype: DataType) -> Optional[_Frag]:
        """``reduce_*`` along the last dimension of a computed tile: the tile's code, then a ROW opcode."""
        src = node.args[0]
        # fp16 / bf16 rows are reduced in fp32 and the result is rounded once (as torch's CPU reductions do)
        if dtype not in (KT.float32, KT.float16, KT.bfloat16) or src.dtype != dtype or node.attrs["kind"] not in _ROW_CODE:
            return None
        dims = node.attrs["dims"]
        if self.full_shape is not None:
            # per-row mode: the reduced tile has the full shape and loses its last dimension
            if src.shape != self.full_shape or dims != (len(src.shape) - 1, ):
                return None
            self.per_row_reductions = True
            outer, outer_full, self.shape, self.full_shape = self.shape, self.full_shape, src.shape, None
            try:
                inner = self.gen(src)
            finally:
                self.shape, self.full_shape = outer, outer_full
        else:
            # the scalar reduction of a whole tile of the stored shape: a single row, or several rows that the
            # row machine walks as one long row (the planner then wants every operand to be a contiguous range)
            rows = 1
            for d in self.shape[:-1]:
                rows *= d
            if dims != () or src.shape != self.shape:
                return None
            if rows != 1:
                self.whole_tile = True
            inner = self.gen(src)
        if inner is None:
            return None
        inner = inner.pushed()
        self.row_ops = True
        return self._rounded(_Frag(inner.code + [(_ROW_CODE[node.attrs["kind"]], 0)], inner.need), dtype)

    def _finish(self, frag: _Frag) -> None:
        """The final program.  In a row program a value that occurs again is computed once: its first occurrence
        is followed by TEE into a temporary slot, every later one is replaced by TMP (the code of a traced value
        does not depend on where it is used).  Elsewhere the markers just drop out."""
        code = frag.pushed().code
        ends = {}
        stack: List[int] = []
        uses: Dict[int, int] = {}
        parent: Dict[int, Optional[int]] = {}     # the value whose code encloses a value's first occurrence
        for i, (op, arg) in enumerate(code):
            if op == _MARK_BEGIN:
                uses[arg] = uses.get(arg, 0) + 1
                parent.setdefault(arg, code[stack[-1]][1] if stack else None)
                stack.append(i)
            elif op == _MARK_END:
                ends[stack.pop()] = i

        def shared(key: int) -> bool:
            # used again on its own, not merely as a part of an enclosing value that is used again
            return uses[key] > (uses[parent[key]] if parent[key] is not None else 1)
        out: List[Tuple[int, int]] = []
        slots: Dict[int, int] = {}
        i = 0
        while i < len(code):
            op, arg = code[i]
            if op == _MARK_BEGIN:
                if self.row_ops and arg in slots:
                    out.append((_OP_TMP, slots[arg]))
                    i = ends[i] + 1
                    continue
            elif op == _MARK_END:
                if self.row_ops and shared(arg) and arg not in slots and len(slots) < ROW_MAX_TMP:
                    slots[arg] = len(slots)
                    out.append((_OP_TEE, slots[arg]))
            else:
                out.append((op, arg))
            i += 1
        self.ops = [c[0] for c in out]
        self.args = [c[1] for c in out]
        self.max_depth = frag.pushed().need
        self.n_tmp = len(slots)

    def compile(self, v: Any) -> bool:
        self.root = v
        frag = self.gen(v)
        if frag is None:
            return False
        self._finish(frag)
        return True


def _tile_windows(tshape: Tuple[int, ...], offsets: Sequence[PlainValue], shape: Tuple[int, ...],
                  env: Dict[str, np.ndarray], n: int):
    """For 2-D tiles of a 2-D tensor: the distinct (row0, col0, rows, cols) windows the instances store, clipped
    to the tensor (stores are clipped, LowerAscTileDataTransfer.cpp:254-261), and whether together they are
    exactly the regular tile grid of the whole tensor."""
    row0, col0 = eval_int(offsets[0], env, n), eval_int(offsets[1], env, n)
    if n and (row0.min() < 0 or col0.min() < 0):
        raise RuntimeError("Negative tile offset in kernel")
    keep = (row0 < tshape[0]) & (col0 < tshape[1])
    origins = sorted(set(zip(row0[keep].tolist(), col0[keep].tolist())))
    windows = [(r, c, min(shape[0], tshape[0] - r), min(shape[1], tshape[1] - c)) for r, c in origins]
    grid = {(r, c) for r in range(0, tshape[0], shape[0]) for c in range(0, tshape[1], shape[1])} \
        if tshape[0] * tshape[1] <= (1 << 24) * shape[0] * shape[1] else None
    return windows, grid is not None and set(origins) == grid


def _flat_scalar_offset(tshape: Tuple[int, ...], offsets: Sequence[PlainValue]) -> PlainValue:
    if len(offsets) != len(tshape):
        raise RuntimeError("number of 'offsets' must match the rank of the tensor")
    flat, stride = PlainValue.const(0), 1
    for d in range(len(tshape) - 1, -1, -1):
        flat = flat + offsets[d] * stride
        stride *= tshape[d]
    return flat


class _Geometry:
    """Where a tile lies in its tensor for every instance: the flat index of its first element and either one
    contiguous range of ``numel`` elements (``pitch`` None) or ``rows`` x ``cols`` with a row pitch."""

    def __init__(self, tensor: Tensor, offsets: Sequence[PlainValue], shape: Tuple[int, ...], scalar: bool,
                 env: Dict[str, np.ndarray], n: int, clip: bool = False):
        """``clip``: a tile may reach past the last row (or the last element of a flat range) of its tensor; how far
        every instance's tile lies inside is kept in ``avail`` (elements of a flat range, rows of a window) for the
        planner to cut the call short, as a clipped store and a padded load of elements nobody stores would."""
        tshape = tensor.static_shape()
        numel = 1
        for d in tshape:
            numel *= d
        self.pitch: Optional[int] = None
        self.rows, self.cols = 1, 1
        self.avail: Optional[np.ndarray] = None
        if scalar:
            self.start = eval_int(_flat_scalar_offset(tshape, offsets), env, n)
            self.numel, ends = 1, None
        else:
            window = _flat_window(tensor, offsets, shape)
            if window is not None:
                self.start = eval_int(window[0], env, n)
                self.numel = window[1]
            elif len(tshape) == 2 and len(shape) == 2:
                r0, c0 = eval_int(offsets[0], env, n), eval_int(offsets[1], env, n)
                if n and (r0.min() < 0 or c0.min() < 0):
                    raise RuntimeError("Negative tile offset in kernel")
                if n and (((r0 + shape[0]).max() > tshape[0] and not clip) or (c0 + shape[1]).max() > tshape[1]):
                    raise _unsupported("tile that reaches past the end of its tensor in a kernel whose operands are "
                                       "addressed differently from its result")
                self.avail = tshape[0] - r0
                self.start = r0 * tshape[1] + c0
                self.rows, self.cols, self.pitch = shape[0], shape[1], tshape[1]
                self.numel = shape[0] * shape[1]
            else:
                raise _unsupported("tile that is neither a contiguous range nor a 2-D window of a matrix")
        if n and self.start.min() < 0:
            raise RuntimeError("Negative tile offset in kernel")
        if self.pitch is None and n and (self.start + self.numel).max() > numel and not (clip and not scalar):
            raise _unsupported("tile that reaches past the end of its tensor in a kernel whose operands are addressed "
                               "differently from its result")
        if self.pitch is None and not scalar:
            self.avail = numel - self.start


def _program_arrays(prog: "_EltProgram", out_t: Tensor):
    n_ops, n_in = len(prog.ops), len(prog.operands)
    return (n_ops, n_in, (ctypes.c_int32 * n_ops)(*prog.ops), (ctypes.c_int32 * n_ops)(*prog.args),
            (ctypes.c_int32 * max(1, n_in))(*[_ELT_TYPE[o.tensor.dtype.name] | (_ROW_SCALAR_INPUT if o.per_row else 0)
                                              for o in prog.operands]), _ELT_TYPE[out_t.dtype.name])


def _program_key(prog: "_EltProgram", row_cols: Optional[int] = None):
    """``(kind, words)`` under which the kernel specialised for this program is built and registered
    (pyasc_b200/jit.py): the launcher asks for it before it runs a step that carries one."""
    from pyasc_b200 import jit
    if not prog.operands:
        return None
    words = jit.program_words(prog.ops, prog.args, [o.per_row for o in prog.operands])
    return (jit.row_kind(row_cols) if row_cols is not None else 0, words)


def _check_program_limits(prog: "_EltProgram") -> None:
    if len(prog.ops) > ELT_MAX_OPS or len(prog.operands) > ELT_MAX_INPUTS or prog.max_depth > ELT_MAX_STACK:
        raise _unsupported(f"elementwise expression with {len(prog.ops)} operations, {len(prog.operands)} inputs and a "
                           f"stack of {prog.max_depth} (limits: {ELT_MAX_OPS}, {ELT_MAX_INPUTS}, {ELT_MAX_STACK})")


def _plan_general_program(trace: KernelTrace, eff: Effect, prog: "_EltProgram", out_t: Tensor,
                          offsets: Sequence[PlainValue], out_shape: Tuple[int, ...], scalar_store: bool,
                          dedupe: bool,
                          row_shape: Optional[Tuple[int, int]] = None, row_result: bool = False) -> Plan:
    """Operands addressed differently from the result (other tensor shapes or offsets, reshapes, a broadcast row,
    an accumulation into a fixed window): one call per (block, iteration) instance, in program order."""
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    if n > MAX_CALLS:
        raise _unsupported("elementwise kernel with differently addressed operands and more than 4096 tiles")
    out_g = _Geometry(out_t, offsets, out_shape, scalar_store, env, n, clip=True)
    geoms = [_Geometry(o.tensor, o.offsets, o.shape, o.scalar, env, n, clip=True) for o in prog.operands]
    # the window every call walks: rows x cols
    rows, cols = (out_g.rows, out_g.cols) if out_g.pitch is not None else (1, out_g.numel)
    for o, g in zip(prog.operands, geoms):
        if out_g.pitch is None and g.pitch is not None and not o.bcast and not o.per_row and g.numel == out_g.numel \
                and tuple(out_shape[-2:]) == (g.rows, g.cols):
            # the result is a contiguous run of rows, an operand a window of a wider matrix (one half of each row,
            # say): the call walks the window's rows x cols, the result with a pitch of one row
            rows, cols = g.rows, g.cols
    for o, g in zip(prog.operands, geoms):
        if o.bcast and out_g.pitch is None and rows == 1:
            if out_g.numel % g.numel:
                raise _unsupported("broadcast of a row whose length does not divide the stored tile")
            rows, cols = out_g.numel // g.numel, g.numel
    if row_shape is not None:
        # a row program walks the rows of the tile as the kernel wrote it: reductions run along them
        rows, cols = row_shape
        kv = 1
        while kv * 256 < cols:
            kv *= 2
        if cols > ROW_MAX_COLS or (max(1, prog.max_depth - 1) + prog.n_tmp) * kv * 1024 > 200 * 1024:
            raise _unsupported(f"row reductions inside an expression over rows of {cols} elements with a stack of "
                               f"{prog.max_depth} (the row and its intermediate values must fit one SM)")
        if out_g.pitch is not None and (out_g.rows, out_g.cols) != (rows, 1 if row_result else cols):
            raise _unsupported("row program stored into a window of a different shape")
        if out_g.pitch is None and out_g.numel != (rows if row_result else rows * cols):
            raise _unsupported("row program stored into a range of a different size")
    if prog.reshaped and (out_g.pitch is not None or any(g.pitch is not None for g in geoms)):
        raise _unsupported("reshape of a tile that is not a contiguous range of its tensor")
    lds: List[int] = []
    for o, g in zip(prog.operands, geoms):
        if o.per_row:
            if g.pitch is None and g.numel == rows:
                lds.append(1)                     # a contiguous [rows] vector
            elif g.pitch is not None and (g.rows, g.cols) == (rows, 1):
                lds.append(g.pitch)               # a column of a matrix
            else:
                raise _unsupported("column operand that does not hold one element per row of the result")
        elif o.bcast:
            if g.numel != cols:
                raise _unsupported("broadcast of a tile that is not one row of the result")
            lds.append(0)
        elif g.pitch is not None:
            if (g.rows, g.cols) != (rows, cols):
                raise _unsupported("operand window of a different shape than the stored tile")
            lds.append(g.pitch)
        else:
            if g.numel != rows * cols:
                raise _unsupported("operand tile with a different number of elements than the stored tile")
            lds.append(cols)
    lds.append(out_g.pitch if out_g.pitch is not None else (1 if row_result else cols))
    out_idx = out_t.base.index
    in_idx = [o.tensor.base.index for o in prog.operands]
    in_size = [o.tensor.dtype.bitwidth // 8 for o in prog.operands]
    out_size = out_t.dtype.bitwidth // 8
    for k, (i, g) in enumerate(zip(in_idx, geoms)):
        # An operand taken from the tensor that is stored to must be the stored window itself, element for element:
        # a thread then reads exactly what it overwrites (`y = x + y` in place, the target of an atomic).
        o = prog.operands[k]
        same_window = (not o.bcast and (not o.per_row or row_result) and not prog.reshaped and lds[k] == lds[-1]
                       and np.array_equal(g.start, out_g.start))
        if i == out_idx and not same_window:
            raise _unsupported("elementwise kernel that stores into a tensor it also loads at other positions")
    plan = Plan("row:program" if row_shape is not None else "elementwise:program")
    plan.reads.update(in_idx)
    plan.writes.add(out_idx)
    plan.partial_writes.add(out_idx)
    n_ops, n_in, ops_arr, args_arr, types_arr, out_type = _program_arrays(prog, out_t)
    lds_arr = (ctypes.c_int64 * len(lds))(*lds)
    fn_name = "asc_cuda_row_program" if row_shape is not None else "asc_cuda_eltwise_program_2d"
    tail_args = (ctypes.c_int32(1 if row_result else 0), ) if row_shape is not None else ()
    program_key = _program_key(prog, cols if row_shape is not None else None)
    # Tiles that reach past the end of their tensors (the last block of a row count that is no multiple of the tile):
    # the store is clipped there, so the call is cut to the rows (for a one-row call: the elements) that exist in the
    # result; every operand must hold at least those, or the kernel would have computed on padding.
    out_cols = 1 if row_result else cols
    full = np.full(n, rows if rows > 1 or row_shape is not None else cols, dtype=np.int64)
    by_rows = rows > 1 or row_shape is not None

    def supply(g: "_Geometry", per_unit: int) -> np.ndarray:
        """Call rows (or, in a one-row call, elements) of each instance's tile that lie inside the tensor."""
        if g.avail is None:
            return full
        if g.pitch is not None:
            return g.avail if by_rows else np.where(g.avail >= 1, full, 0)
        return g.avail // per_unit if by_rows else g.avail
    have = np.minimum(full, np.maximum(supply(out_g, out_cols), 0))
    if by_rows and out_g.pitch is None and out_g.avail is not None and np.any((np.minimum(out_g.avail, out_g.numel) % out_cols) != 0):
        raise _unsupported("tile whose part inside the tensor is not a whole number of rows")
    for o, g in zip(prog.operands, geoms):
        if o.bcast or o.scalar:
            if g.avail is not None and np.any(g.avail < (g.numel if g.pitch is None else g.rows)):
                raise _unsupported("broadcast row that reaches past the end of its tensor (zero padding)")
            continue
        if np.any(supply(g, 1 if o.per_row else cols) < have):
            raise _unsupported("operand tile that reaches past the end of its tensor where the result does not "
                               "(zero padding would be computed on)")
    calls: List[Tuple[Tuple[int, ...], int, int]] = []  # (first element of every operand and of the result, rows, cols)
    keep = [j for j in range(n) if have[j] > 0]
    extent = {}
    all_starts = []
    for j in keep:
        st = tuple(int(g.start[j]) for g in geoms) + (int(out_g.start[j]), )
        all_starts.append(st)
        extent[st] = max(extent.get(st, 0), int(have[j]))
    if dedupe and len(set(all_starts)) > 1:
        # Instances that differ in where they read from but write overlapping elements do not commute: the last
        # writer (in block order, then iteration order) must win, so such a kernel keeps one call per instance in
        # that order.  Instances with equal addresses throughout are repeats of one another.
        uniq = sorted(set(all_starts))
        u = np.array(uniq, dtype=np.int64)
        width = out_t.static_shape()[-1] if out_t.static_shape() else 1
        if out_g.pitch is None:
            # flat ranges, cut at the end of the tensor where a tile reaches past it
            ends = np.minimum(u[:, -1] + out_g.numel, out_t.base.numel)
            rect = np.stack([np.zeros_like(ends), np.ones_like(ends), u[:, -1], ends], axis=1)
        else:
            rect = _flat_rects(width, u[:, -1], out_g.numel, out_g.rows, out_g.cols, out_g.pitch)
        clash = _rects_overlap(rect, rect)
        np.fill_diagonal(clash, False)
        if clash.any():
            dedupe = False
    if dedupe:
        # stores are idempotent and independent: drop repeats, and let windows that continue each other row
        # after row (every operand advancing by its own pitch, a broadcast row staying put) become one call
        for starts in sorted(set(all_starts), key=lambda st: st[-1]):
            here = (extent[starts], cols) if by_rows else (rows, extent[starts])
            if calls and cols > 0 and not prog.uses_index:      # (an element index restarts with every tile)
                prev, prev_rows, prev_cols = calls[-1]
                if prev_cols == here[1] and all(st == p0 + prev_rows * ld for st, p0, ld in zip(starts, prev, lds)):
                    calls[-1] = (prev, prev_rows + here[0], prev_cols)
                    continue
            calls.append((starts, ) + here)
    else:
        calls = [(all_starts[k], int(have[j]), cols) if by_rows else (all_starts[k], rows, int(have[j]))
                 for k, j in enumerate(keep)]

    def make_step(starts: Tuple[int, ...], call_rows: int, call_cols: int = cols) -> Step:
        def build(ptrs, stream):
            ins = (ctypes.c_void_p * max(1, n_in))(*[ptrs[i] + sz * st for i, sz, st in zip(in_idx, in_size, starts)])
            return (ops_arr, args_arr, ctypes.c_int32(n_ops), ins, types_arr, ctypes.c_int32(n_in),
                    _p(ptrs[out_idx] + out_size * starts[-1]), ctypes.c_int32(out_type), ctypes.c_int64(call_rows),
                    ctypes.c_int64(call_cols), lds_arr) + tail_args + (stream, )
        step = Step(fn_name, build,
                    f"{n_ops} ops over [{call_rows}, {call_cols}] pitches {lds} from {list(starts[:-1])} to {starts[-1]}")
        step.program, step.elements = program_key, call_rows * call_cols
        return step

    for starts, call_rows, call_cols in calls:
        plan.steps.append(make_step(starts, call_rows, call_cols))
    covered = sum(r * (1 if row_result else c) for _, r, c in calls)
    if dedupe and len(calls) == 1 and lds[-1] == out_cols and calls[0][0][-1] == 0 and covered == out_t.base.numel:
        plan.partial_writes.discard(out_idx)
    if not plan.steps:
        return plan          # no block has a tile inside the tensors (an empty tensor): nothing to launch
    if row_shape is not None and not plan.partial_writes and len(calls) == 1:
        # whole rows of whole tensors: chunks of rows can be uploaded, computed and downloaded independently;
        # a broadcast row is needed by every chunk
        starts0, total_rows, _ = calls[0]
        whole = all(st == 0 and (ld == 0 or ld * total_rows == o.tensor.base.numel)
                    for st, ld, o in zip(starts0, lds, prog.operands))
        if whole and len(set(in_idx)) == len(in_idx) and out_idx not in in_idx:
            streamed = {i: sz * ld for i, sz, ld in zip(in_idx, in_size, lds) if ld != 0}
            streamed[out_idx] = out_size * lds[-1]
            resident = {i for i, ld in zip(in_idx, lds) if ld == 0}
            plan.pipeline = PipelineSpec(total_rows, 1, streamed, resident,
                                         lambda lo, hi: [make_step(tuple(lo * ld for ld in lds), hi - lo)])
    return plan


def _twin_key(tensor: Tensor) -> str:
    return f"wide{tensor.base.index}"


def _fake_like(key: str, tensor: Tensor, dtype: DataType) -> Tensor:
    """A temporary of ``tensor``'s shape and another element type."""
    from ..language.core.ir_value import GlobalAddress
    base = GlobalAddress(key, dtype, key, tensor.base.numel)  # type: ignore[arg-type]
    return Tensor(base, tuple(PlainValue.const(d) for d in tensor.static_shape()))


def _convert_step(dst: Any, src: Any, n: int, mode: int, note: str) -> Step:
    def build(ptrs, stream):
        return (_p(ptrs[dst]), _p(ptrs[src]), ctypes.c_int64(n), ctypes.c_int32(mode), stream)
    return Step("asc_cuda_convert_bytes", build, note)


def _match_eltwise_program(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """An elementwise or row program.  int8 / uint8 tensors take part through int32 twins: every 8-bit tensor the
    program loads is widened, whole, into a temporary first; an 8-bit result (an int32 value cast down) is computed
    into the twin of the output tensor and narrowed out of it afterwards -- the twin is filled from the tensor
    first where the kernel writes only part of it, so that the rest keeps its bytes."""
    value, out_t = eff.args
    narrow = None
    if out_t.dtype.name in _BYTE_TYPES:
        cast = _node(value, "cast") if isinstance(value, Tile) else None
        if cast is None or value.dtype != out_t.dtype or cast.args[0].dtype != KT.int32:
            return None          # (a loaded 8-bit tile stored as it is: a copy)
        narrow = (_fake_like(_twin_key(out_t), out_t, KT.int32), out_t)
        eff = Effect(eff.kind, (cast.args[0], narrow[0]), eff.attrs, eff.loops, eff.guards)
    found = _plan_eltwise_program(trace, eff)
    if found is None:
        return None
    plan, prog = found
    if not prog.twins and narrow is None:
        return plan
    before: List[Step] = []
    for key, (twin, real) in prog.twins.items():
        if narrow is not None and real.base.index == narrow[1].base.index:
            raise _unsupported("8-bit tensor that a kernel both loads and stores")
        plan.temps[key] = 4 * real.base.numel
        before.append(_convert_step(key, real.base.index, real.base.numel, 0 if real.dtype.name == "int8" else 1,
                                    f"{real.dtype.name}[{real.base.numel}] -> int32 temporary"))
        plan.reads.discard(key)
        plan.reads.add(real.base.index)
    after: List[Step] = []
    if narrow is not None:
        twin, real = narrow
        key, idx, n = twin.base.index, real.base.index, real.base.numel
        plan.temps[key] = 4 * n
        if key in plan.partial_writes:
            before.append(_convert_step(key, idx, n, 0 if real.dtype.name == "int8" else 1,
                                        f"{real.dtype.name}[{n}] -> int32 temporary (the part the kernel leaves)"))
            plan.partial_writes.discard(key)
            plan.partial_writes.add(idx)
        after.append(_convert_step(idx, key, n, 2, f"int32 temporary -> {real.dtype.name}[{n}]"))
        plan.writes.discard(key)
        plan.writes.add(idx)
    plan.steps = before + plan.steps + after
    plan.pipeline = None
    return plan


def _plan_eltwise_program(trace: KernelTrace, eff: Effect) -> Optional[Tuple[Plan, "_EltProgram"]]:
    plan_prog: List[Any] = []
    plan = _plan_eltwise_program_with(trace, eff, plan_prog)
    return None if plan is None else (plan, plan_prog[0])


def _plan_eltwise_program_with(trace: KernelTrace, eff: Effect, made: List[Any]) -> Optional[Plan]:
    value, out_t = eff.args
    offsets = eff.attrs["offsets"]
    scalar_store = eff.kind == "store_scalar"
    if not isinstance(value, (Tile, PlainValue)) or out_t.dtype.name not in _ELT_TYPE or value.dtype != out_t.dtype:
        return None
    tshape = out_t.static_shape()
    out_shape = (1, ) if scalar_store else value.shape
    prog = _EltProgram(out_shape, offsets, out_t, scalar_store)
    prog.allow_bytes = True
    made.append(prog)
    if not prog.compile(value):
        return None
    _check_program_limits(prog)
    _check_fits(out_t)
    for t in prog.inputs:
        _check_fits(t)
    if scalar_store:
        aligned = all(o.scalar and o.tensor.static_shape() == tshape and _same_offsets(o.offsets, offsets)
                      for o in prog.operands)
    else:
        aligned = not prog.reshaped and not prog.uses_index and \
            all(o.addressed_like(out_t, offsets, out_shape) for o in prog.operands)
    if prog.row_ops:
        rows = 1
        for d in out_shape[:-1]:
            rows *= d
        if prog.whole_tile:
            if prog.per_row_reductions or prog.uses_index:
                raise _unsupported("reductions of a whole tile and along its rows in one expression")
            return _plan_general_program(trace, eff, prog, out_t, offsets, out_shape, False, dedupe=True,
                                         row_shape=(1, rows * out_shape[-1]))
        return _plan_general_program(trace, eff, prog, out_t, offsets, out_shape, False, dedupe=True,
                                     row_shape=(rows, out_shape[-1]))
    if not aligned or not prog.operands:
        return _plan_general_program(trace, eff, prog, out_t, offsets, out_shape, scalar_store, dedupe=True)
    numel = 1
    for d in tshape:
        numel *= d
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    windows: List[Tuple[int, int, int, int]] = []     # 2-D mode: (row0, col0, rows, cols)
    if scalar_store:
        window = (_flat_scalar_offset(tshape, offsets), 1)
    else:
        window = _flat_window(out_t, offsets, value.shape)
    if window is not None:
        flat_off, tile_elems = window
        starts = eval_int(flat_off, env, n)
        if starts.size and starts.min() < 0:
            raise RuntimeError("Negative tile offset in kernel")
        intervals = merge_intervals(starts, np.minimum(starts + tile_elems, numel))
    elif len(tshape) == 2 and len(value.shape) == 2:
        windows, whole = _tile_windows(tshape, offsets, value.shape, env, n)
        intervals = [(0, numel)] if whole else []
        if whole:
            windows = []
    else:
        raise _unsupported("elementwise kernel whose tiles are neither contiguous ranges nor 2-D windows of a matrix")
    if len(intervals) + len(windows) > MAX_CALLS:
        raise _unsupported("elementwise kernel touching more than 4096 disjoint ranges")

    plan = Plan("elementwise:program")
    out_idx = out_t.base.index
    in_idx = [t.base.index for t in prog.inputs]
    in_size = [t.dtype.bitwidth // 8 for t in prog.inputs]
    out_size = out_t.dtype.bitwidth // 8
    if out_idx in in_idx:
        raise _unsupported("elementwise kernel that stores into a tensor it also loads")
    plan.reads.update(in_idx)
    plan.writes.add(out_idx)
    if intervals != [(0, out_t.base.numel)]:
        plan.partial_writes.add(out_idx)
    n_ops, n_in, ops_arr, args_arr, types_arr, out_type = _program_arrays(prog, out_t)
    program_key = _program_key(prog)

    def make(lo: int, hi: int) -> List[Step]:
        def build(ptrs, stream, lo=lo, hi=hi):
            # the library copies the program and the pointer table before it returns
            ins = (ctypes.c_void_p * n_in)(*[ptrs[i] + sz * lo for i, sz in zip(in_idx, in_size)])
            return (ops_arr, args_arr, ctypes.c_int32(n_ops), ins, types_arr, ctypes.c_int32(n_in),
                    _p(ptrs[out_idx] + out_size * lo), ctypes.c_int32(out_type), ctypes.c_int64(hi - lo), stream)
        step = Step("asc_cuda_eltwise_program", build, f"{n_ops} ops over [{lo}, {hi})")
        step.program, step.elements = program_key, hi - lo
        return [step]

    lds_arr = (ctypes.c_int64 * (n_in + 1))(*([tshape[-1]] * (n_in + 1)))

    def make_2d(r0: int, c0: int, rows: int, cols: int) -> Step:
        first = r0 * tshape[1] + c0

        def build(ptrs, stream):
            ins = (ctypes.c_void_p * n_in)(*[ptrs[i] + sz * first for i, sz in zip(in_idx, in_size)])
            return (ops_arr, args_arr, ctypes.c_int32(n_ops), ins, types_arr, ctypes.c_int32(n_in),
                    _p(ptrs[out_idx] + out_size * first), ctypes.c_int32(out_type), ctypes.c_int64(rows),
                    ctypes.c_int64(cols), lds_arr, stream)
        step = Step("asc_cuda_eltwise_program_2d", build, f"{n_ops} ops over [{rows}, {cols}] at ({r0}, {c0})")
        step.program, step.elements = program_key, rows * cols
        return step

    for lo, hi in intervals:
        plan.steps += make(lo, hi)
    for w in windows:
        plan.steps.append(make_2d(*w))
    if not plan.steps:
        return plan          # no block has a tile inside the tensor (an empty tensor): nothing to launch
    if not plan.partial_writes and len(intervals) == 1:
        streamed = {i: sz for i, sz in zip(in_idx, in_size)}
        streamed[out_idx] = out_size
        plan.pipeline = PipelineSpec(intervals[0][1], 1 << 16, streamed, set(), make)
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: atomic accumulation of a tile into a window of a tensor (add / max / min)
# --------------------------------------------------------------------------------------------------
def _match_atomic(trace: KernelTrace, eff: Effect) -> Plan:
    """``asc2.atomic_add/max/min(tile, tensor, offsets)``: tensor[window] = op(tensor[window], tile).  The blocks'
    accumulations are applied one after the other on the launch stream, in block order, so the result is the
    one any serial order of the reference's atomics gives (exactly for max / min and integers, within fp
    rounding for floating-point sums)."""
    value, out_t = eff.args
    offsets = eff.attrs["offsets"]
    if not isinstance(value, Tile) or out_t.dtype.name not in _ELT_TYPE or value.dtype != out_t.dtype:
        raise _unsupported(f"atomic_{eff.attrs['kind']} of a {getattr(value, 'dtype', type(value).__name__)} tile into a "
                           f"{out_t.dtype} tensor")
    table = _BINARY_CODE if out_t.dtype.is_float() else _INT_BINARY_CODE
    prog = _EltProgram(value.shape, offsets, out_t)
    current = prog._load(_Operand(out_t, offsets, value.shape))
    update = prog.gen(value)
    row_shape = None
    if current is None or update is None or prog.row_ops:
        # one value per row, computed from reductions along the rows of a tile (partial row sums of a column block
        # accumulated into a vector): a row program that loads the target element of its row and stores it back
        red = _find_row_reduction(value)
        full_shape = red.args[0].shape if red is not None else None
        if red is None or value.shape not in ((full_shape[0], ), (full_shape[0], 1)) or not out_t.dtype.is_float():
            raise _unsupported("atomic operation on a tile that is neither an elementwise expression of loaded tiles nor "
                               "one value per row of a tile reduced along its rows")
        prog = _EltProgram(value.shape, offsets, out_t)
        update = prog._per_row(value, full_shape)
        current = prog._load(_Operand(out_t, offsets, value.shape, per_row=True))
        if update is None or current is None or not prog.row_ops:
            raise _unsupported("atomic operation on an expression of row reductions that is not expressible")
        row_shape = (full_shape[0], full_shape[1])
    prog._finish(prog._rounded(prog._binary(table[eff.attrs["kind"]], current, update), out_t.dtype))
    _check_program_limits(prog)
    _check_fits(out_t)
    for t in prog.inputs:
        _check_fits(t)
    if row_shape is not None:
        plan = _plan_general_program(trace, eff, prog, out_t, offsets, value.shape, False, dedupe=False,
                                     row_shape=row_shape, row_result=True)
    else:
        plan = _plan_general_program(trace, eff, prog, out_t, offsets, value.shape, False, dedupe=False)
    plan.pattern = f"atomic:{eff.attrs['kind']}"
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: one value per row, computed from reductions of elementwise expressions along the row
# --------------------------------------------------------------------------------------------------
def _find_row_reduction(v: Any, depth: int = 0, seen: Optional[set] = None) -> Optional[Node]:
    """The first reduction along the last dimension of a 2-D tile in the expression graph of ``v``."""
    seen = set() if seen is None else seen
    if depth > 64 or id(v) in seen:
        return None
    seen.add(id(v))
    if isinstance(v, PlainValue):
        args = v.args if v.op not in ("const", "sym") else ()
    elif isinstance(v, Tile):
        node = v.node
        if node.kind == "reduce" and len(node.args[0].shape) == 2 and node.attrs["dims"] == (1, ):
            return node
        args = node.args
    elif isinstance(v, Node):
        args = v.args
    else:
        return None
    for a in args:
        found = _find_row_reduction(a, depth + 1, seen)
        if found is not None:
            return found
    return None


def _match_row_result(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(f(reduce(g(tiles), 1), ...), vector)``: a [rows] (or [rows, 1]) tile whose elements are functions of
    row reductions of computed tiles, e.g. ``reduce_sum(x * x, 1)``.  One row program, one stored element per row."""
    value, out_t = eff.args
    # (a tile of one element, the reduction of a one-row tile, arrives as a scalar store)
    if not isinstance(value, Tile) or eff.kind not in ("store", "store_scalar") or value.dtype != out_t.dtype or \
            value.dtype not in (KT.float32, KT.float16, KT.bfloat16):
        return None
    direct = _node(value, "reduce")
    if direct is not None and direct.args[0].node.kind in ("load", "copy") and value.dtype == KT.float32:
        return None                        # a reduction of a loaded fp32 tile has its own kernel
    red = _find_row_reduction(value)
    if red is None:
        return None
    full_shape = red.args[0].shape
    if value.shape not in ((full_shape[0], ), (full_shape[0], 1)):
        return None
    offsets = eff.attrs["offsets"]
    prog = _EltProgram(value.shape, offsets, out_t)
    frag = prog._per_row(value, full_shape)
    if frag is None or not prog.row_ops:
        return None
    prog._finish(frag)
    _check_program_limits(prog)
    _check_fits(out_t)
    for t in prog.inputs:
        _check_fits(t)
    return _plan_general_program(trace, eff, prog, out_t, offsets, value.shape, eff.kind == "store_scalar", dedupe=True,
                                 row_shape=(full_shape[0], full_shape[1]), row_result=True)


def _find_scalar_reduction(v: Any, depth: int = 0) -> Optional[Node]:
    """The first whole-tile reduction in the expression tree of the scalar ``v``."""
    if depth > 64 or not isinstance(v, PlainValue) or v.op in ("const", "sym"):
        return None
    if v.op == "tile_scalar":
        node = v.args[0]
        return node if node.kind == "reduce" and node.attrs["dims"] == () else None
    for a in v.args:
        found = _find_scalar_reduction(a, depth + 1)
        if found is not None:
            return found
    return None


def _match_row_scalar(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(f(reduce(g(row))), tensor, offsets)``: one element computed from whole-tile reductions of an
    elementwise expression over a one-row tile (also wrapped in ``asc2.full([1], ...)``, the reference's idiom for
    storing a scalar).  A row program over that row with one stored element."""
    value, out_t = eff.args
    if eff.kind != "store_scalar" or out_t.dtype != KT.float32:
        return None
    v = value
    if isinstance(v, Tile):
        full = _node(v, "full")
        if full is None:
            return None
        v = full.attrs["value"]
    if not isinstance(v, PlainValue) or v.is_const or v.dtype != KT.float32:
        return None
    red = _find_scalar_reduction(v)
    if red is None:
        return None
    src = red.args[0]
    rows = 1
    for d in src.shape[:-1]:
        rows *= d
    if rows != 1:
        return None
    if v.op == "tile_scalar" and v.args[0] is red and src.node.kind in ("load", "copy"):
        return None                        # a reduction of a loaded tile has its own kernel
    offsets = eff.attrs["offsets"]
    prog = _EltProgram(src.shape, offsets, out_t)
    frag = prog.gen(v, KT.float32)
    if frag is None or not prog.row_ops:
        return None
    prog._finish(frag)
    _check_program_limits(prog)
    _check_fits(out_t)
    for t in prog.inputs:
        _check_fits(t)
    return _plan_general_program(trace, eff, prog, out_t, offsets, (1, ), True, dedupe=True,
                                 row_shape=(1, src.shape[-1]), row_result=True)


# --------------------------------------------------------------------------------------------------
# Pattern: reduction of a loaded tile along one axis, or of the whole tile broadcast into the store
# --------------------------------------------------------------------------------------------------
_REDUCE_KIND = {"sum": 0, "max": 1, "min": 2, "prod": 3}


def _match_col_reduce(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(reduce_*(expression, 0), vector)``: a 2-D tile that is computed (or loaded as fp16 / bf16) and reduced
    along its first dimension: one column program per tile, a thread per column (``asc_cuda_col_program``).  A loaded
    fp32 tile keeps the dedicated reduction kernel."""
    value, out_t = eff.args
    node = _node(value, "reduce") if isinstance(value, Tile) and eff.kind == "store" else None
    if node is None or node.attrs["dims"] != (0, ):
        return None
    src = node.args[0]
    dtype = value.dtype
    if len(src.shape) != 2 or dtype not in (KT.float32, KT.float16, KT.bfloat16) or src.dtype != dtype or out_t.dtype != dtype:
        return None
    if src.node.kind in ("load", "copy") and dtype == KT.float32:
        return None
    rows, cols = src.shape
    if value.shape not in ((cols, ), (1, cols)) or node.attrs["kind"] not in _REDUCE_KIND:
        return None
    offsets = eff.attrs["offsets"]
    prog = _EltProgram(src.shape, offsets, out_t)
    frag = prog.gen(src)
    if frag is None or prog.row_ops or prog.reshaped:
        return None
    prog._finish(frag)
    _check_program_limits(prog)
    _check_fits(out_t)
    for t in prog.inputs:
        _check_fits(t)
    window = _flat_window(out_t, offsets, value.shape)
    if window is None:
        raise _unsupported("column reduction whose result is not stored as one contiguous range")
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    if n > MAX_CALLS:
        raise _unsupported("column reduction of a computed tile in more than 4096 tiles")
    out0 = eval_int(window[0], env, n)
    if n and (out0.min() < 0 or (out0 + cols).max() > out_t.base.numel):
        raise _unsupported("column reduction whose result reaches past the end of its tensor")
    geoms = [_Geometry(o.tensor, o.offsets, o.shape, o.scalar, env, n) for o in prog.operands]
    lds: List[int] = []
    for o, g in zip(prog.operands, geoms):
        if o.bcast:
            if g.numel != cols:
                raise _unsupported("broadcast of a tile that is not one row of the reduced tile")
            lds.append(0)
        elif g.pitch is not None:
            if (g.rows, g.cols) != (rows, cols):
                raise _unsupported("operand window of a different shape than the reduced tile")
            lds.append(g.pitch)
        else:
            if g.numel != rows * cols:
                raise _unsupported("operand tile with a different number of elements than the reduced tile")
            lds.append(cols)
    out_idx = out_t.base.index
    in_idx = [o.tensor.base.index for o in prog.operands]
    if out_idx in in_idx:
        raise _unsupported("column reduction that stores into a tensor it loads")
    calls = sorted(set(tuple(int(g.start[j]) for g in geoms) + (int(out0[j]), ) for j in range(n)), key=lambda c: c[-1])
    if any(b[-1] < a[-1] + cols for a, b in zip(calls, calls[1:])):
        raise _unsupported("column reductions of different tiles stored into overlapping ranges (the last writer would win)")
    if not calls:
        raise _unsupported("column reduction without any tile")
    in_size = [o.tensor.dtype.bitwidth // 8 for o in prog.operands]
    out_size = out_t.dtype.bitwidth // 8
    n_ops, n_in, ops_arr, args_arr, types_arr, out_type = _program_arrays(prog, out_t)
    lds_arr = (ctypes.c_int64 * max(1, len(lds)))(*lds)
    kind = _REDUCE_KIND[node.attrs["kind"]]
    plan = Plan(f"reduce:{node.attrs['kind']}:columns")
    plan.reads.update(in_idx)
    plan.writes.add(out_idx)
    covered = calls[0][-1] == 0 and all(b[-1] == a[-1] + cols for a, b in zip(calls, calls[1:]))
    if not (covered and calls[-1][-1] + cols == out_t.base.numel):
        plan.partial_writes.add(out_idx)

    def make_step(starts: Tuple[int, ...]) -> Step:
        def build(ptrs, stream):
            ins = (ctypes.c_void_p * max(1, n_in))(*[ptrs[i] + sz * st for i, sz, st in zip(in_idx, in_size, starts)])
            return (ops_arr, args_arr, ctypes.c_int32(n_ops), ins, types_arr, ctypes.c_int32(n_in),
                    _p(ptrs[out_idx] + out_size * starts[-1]), ctypes.c_int32(out_type), ctypes.c_int64(rows),
                    ctypes.c_int64(cols), lds_arr, ctypes.c_int32(kind), stream)
        return Step("asc_cuda_col_program", build,
                    f"{node.attrs['kind']} over the rows of {n_ops} ops on [{rows}, {cols}] from {list(starts[:-1])} to {starts[-1]}")

    for starts in calls:
        plan.steps.append(make_step(starts))
    return plan


def _match_reduce(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    value, out_t = eff.args
    offsets = eff.attrs["offsets"]
    if not isinstance(value, Tile):
        return None
    node = _node(value, "reduce")
    n_fill = 0
    if node is None:
        full = _node(value, "full")
        node = _tile_scalar_node(full.attrs["value"], "reduce") if full is not None else None
        if node is None or node.attrs["dims"] != ():
            return None
        n_fill = value.size
    src = node.args[0]
    view = resolve_view(src) if _node(src, "load") or _node(src, "copy") else None
    if view is None:
        raise _unsupported("reduction of a tile that is not loaded from global memory")
    dtype = src.dtype
    if dtype not in (KT.float32, KT.float16, KT.bfloat16) or out_t.dtype != dtype or view.tensor.dtype != dtype:
        raise _unsupported(f"reduction of {src.dtype} tiles (float32 only; float16 and bfloat16 along one axis or of a whole tile)")
    if len(view.shape) > 2:
        raise _unsupported("reduction of a tile of rank > 2")
    _check_fits(out_t)
    _check_fits(view.tensor)
    x_rows, x_cols = _row_major_2d(view.tensor)
    t_rows, t_cols = (1, view.shape[0]) if len(view.shape) == 1 else view.shape
    dims = node.attrs["dims"]
    if n_fill or len(view.shape) == 1:
        if dims not in ((), (0, )):
            raise _unsupported("reduction axis of a 1-D tile")
        axis, n_out = -1, (n_fill or 1)
    else:
        if len(dims) != 1:
            raise _unsupported("reduction over several axes at once")
        axis = dims[0]
        n_out = t_rows if axis == 1 else t_cols
    if value.size != n_out:
        return None
    if dtype != KT.float32 and axis != -1:        # (loaded 16-bit tiles along an axis are row / column programs)
        raise _unsupported(f"reduction of {src.dtype} tiles along an axis in this form")
    window = _flat_window(out_t, offsets, value.shape)
    if window is None:
        raise _unsupported("reduction whose result is not stored as one contiguous range")
    out_off_expr, out_elems = window
    assert out_elems == n_out
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    zero = PlainValue.const(0)
    x_offs = view.offsets if len(view.offsets) == 2 else (zero, view.offsets[0])
    row0, col0 = eval_int(x_offs[0], env, n), eval_int(x_offs[1], env, n)
    out0 = eval_int(out_off_expr, env, n)
    if n and (row0.min() < 0 or col0.min() < 0 or out0.min() < 0):
        raise RuntimeError("Negative tile offset in kernel")
    if n and ((row0 + t_rows).max() > x_rows or (col0 + t_cols).max() > x_cols):
        raise _unsupported("reduction of a tile that reaches past the end of its tensor")
    if n and (out0 + n_out).max() > out_t.base.numel:
        raise _unsupported("reduction whose result reaches past the end of its tensor")
    if n > (1 << 20):
        raise _unsupported(f"reduction kernel with {n} tiles; use larger tiles")
    calls = sorted(set(zip(row0.tolist(), col0.tolist(), out0.tolist())))
    by_out = sorted(c[2] for c in calls)
    if any(b < a + n_out for a, b in zip(by_out, by_out[1:])):
        raise _unsupported("reductions of different tiles stored into overlapping ranges (the last writer would win)")
    # full-row tiles reduced along the row: consecutive tiles merge into one call over more rows
    merged: List[Tuple[int, int, int, int]] = []      # (row0, col0, out0, rows)
    for r0, c0, o0 in calls:
        if merged and axis == 1 and t_cols == x_cols:
            pr, pc, po, prow = merged[-1]
            if r0 == pr + prow and o0 == po + prow:
                merged[-1] = (pr, pc, po, prow + t_rows)
                continue
        merged.append((r0, c0, o0, t_rows))
    if len(merged) > MAX_CALLS:
        raise _unsupported("reduction kernel that needs more than 4096 separate calls")
    plan = Plan(f"reduce:{node.attrs['kind']}")
    x_idx, out_idx = view.tensor.base.index, out_t.base.index
    if x_idx == out_idx:
        raise _unsupported("reduction that stores into the tensor it loads")
    plan.reads.add(x_idx)
    plan.writes.add(out_idx)
    covered = merge_intervals(np.array([m[2] for m in merged]), np.array([m[2] + (m[3] if axis == 1 else n_out) for m in merged]))
    if covered != [(0, out_t.base.numel)]:
        plan.partial_writes.add(out_idx)
    kind = _REDUCE_KIND[node.attrs["kind"]]

    esize = dtype.bitwidth // 8

    def make_step(r0: int, c0: int, o0: int, rows: int) -> Step:
        note = (f"{node.attrs['kind']} axis {axis} of [{rows}, {t_cols}] at ({r0}, {c0}) -> "
                f"[{o0}, +{rows if axis == 1 else n_out})")
        if dtype != KT.float32:          # a whole 16-bit tile: fp32 combination, one rounding
            def build16(ptrs, stream):
                return (_p(ptrs[x_idx] + esize * (r0 * x_cols + c0)), _p(ptrs[out_idx] + esize * o0), ctypes.c_int64(rows),
                        ctypes.c_int64(t_cols), ctypes.c_int64(x_cols), ctypes.c_int32(kind), ctypes.c_int64(n_fill or 1),
                        ctypes.c_int32(1 if dtype == KT.bfloat16 else 0), stream)
            return Step("asc_cuda_reduce_all_f16", build16, note)

        def build(ptrs, stream):
            return (_p(ptrs[x_idx] + 4 * (r0 * x_cols + c0)), _p(ptrs[out_idx] + 4 * o0), ctypes.c_int64(rows),
                    ctypes.c_int64(t_cols), ctypes.c_int64(x_cols), ctypes.c_int32(axis), ctypes.c_int32(kind),
                    ctypes.c_int64(n_fill or 1), stream)
        return Step("asc_cuda_reduce_f32", build, note)

    for r0, c0, o0, rows in merged:
        plan.steps.append(make_step(r0, c0, o0, rows))
    if len(merged) == 1 and axis == 1 and merged[0][:3] == (0, 0, 0) and t_cols == x_cols and not plan.partial_writes \
            and merged[0][3] * x_cols == view.tensor.base.numel:
        # whole rows of the whole tensor: chunks of rows can be uploaded, reduced and downloaded independently
        plan.pipeline = PipelineSpec(merged[0][3], 64, {x_idx: 4 * x_cols, out_idx: 4}, set(),
                                     lambda lo, hi: [make_step(lo, 0, lo, hi - lo)])
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: row softmax (manual reduce_max / exp / reduce_sum form, and asc2.softmax)
# --------------------------------------------------------------------------------------------------
def _softmax_source(value: Tile) -> Optional[Tile]:
    """The tile X such that ``value == softmax(X)`` over all of X's elements per row, or None."""
    sm = _node(value, "softmax")
    if sm is not None:
        return sm.args[0]
    div = _node(value, "binary", op="div")
    if div is None:
        return None
    numer, denom = div.args
    rs = _tile_scalar_node(denom, "reduce", kind="sum")
    if rs is None or not isinstance(numer, Tile) or rs.args[0].node is not numer.node:
        return None
    ex = _node(numer, "unary", op="exp")
    if ex is None:
        return None
    sub = _node(ex.args[0], "binary", op="sub")
    if sub is None:
        return None
    row, mx = sub.args
    rm = _tile_scalar_node(mx, "reduce", kind="max")
    if rm is None or not isinstance(row, Tile) or rm.args[0].node is not row.node:
        return None
    # the no-axis reductions span the whole tile, so this equals a row softmax only for 1-row tiles
    rows = 1
    for d in row.shape[:-1]:
        rows *= d
    if rows != 1:
        return None
    return row


def _match_softmax(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    value, out_t = eff.args
    if not isinstance(value, Tile):
        return None
    src = _softmax_source(value)
    if src is None:
        return None
    view = resolve_view(src) if _node(src, "load") or _is_materialised(src) else None
    if view is None:
        if _MATERIALISED:
            raise _unsupported("softmax of a tile that is not loaded directly from global memory")
        # a matmul result (_match_matmul_then_program writes it to a temporary and comes back) or another computed
        # tile (a row program computes exp(x - max) / sum over it)
        return None
    if not _same_offsets(view.offsets, eff.attrs["offsets"]) or view.shape != value.shape:
        raise _unsupported("softmax stored at a different position than it was loaded from")
    if value.dtype not in (KT.float32, KT.float16) or out_t.dtype != value.dtype or view.tensor.dtype != value.dtype:
        raise _unsupported(f"softmax on {value.dtype} tiles (float32 and float16 only)")
    esize = value.dtype.bitwidth // 8
    fn_name = "asc_cuda_softmax_f32" if value.dtype == KT.float32 else "asc_cuda_softmax_f16"
    if view.tensor.static_shape() != out_t.static_shape():
        raise _unsupported("softmax between tensors of different shapes")
    _check_fits(out_t)
    _check_fits(view.tensor)
    R, C = _row_major_2d(out_t)
    tile_rows = 1 if len(value.shape) == 1 else value.shape[0]
    tile_cols = value.shape[-1]
    if len(value.shape) == 1:
        row_off, col_off = PlainValue.const(0), view.offsets[0]
    else:
        row_off, col_off = view.offsets
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    r0 = eval_int(row_off, env, n)
    c0 = eval_int(col_off, env, n)
    if n and (r0.min() < 0 or c0.min() < 0):
        raise RuntimeError("Negative tile offset in kernel")
    if n and not np.all(c0 == c0[0]):
        raise _unsupported("softmax tiles at varying column offsets")
    col0 = int(c0[0]) if n else 0
    if col0 + tile_cols > C:
        # the reference pads the load with zeros, which then take part in max and sum
        raise _unsupported("softmax tile wider than the tensor row (zero padding would enter the softmax)")
    intervals = merge_intervals(r0, np.minimum(r0 + tile_rows, R))
    if len(intervals) > MAX_CALLS:
        raise _unsupported("softmax kernel touching more than 4096 disjoint row ranges")
    plan = Plan("softmax")
    in_idx, out_idx = view.tensor.base.index, out_t.base.index
    plan.reads.add(in_idx)
    plan.writes.add(out_idx)
    if not (intervals == [(0, R)] and col0 == 0 and tile_cols == C and R * C == out_t.base.numel):
        plan.partial_writes.add(out_idx)
    def make(lo: int, hi: int) -> List[Step]:
        def build(ptrs, stream, lo=lo, hi=hi):
            byte_off = esize * (lo * C + col0)
            return (_p(ptrs[in_idx] + byte_off), _p(ptrs[out_idx] + byte_off), ctypes.c_int64(hi - lo),
                    ctypes.c_int64(tile_cols), ctypes.c_int64(C), stream)
        return [Step(fn_name, build, f"rows [{lo}, {hi}) x {tile_cols} cols")]

    for lo, hi in intervals:
        plan.steps += make(lo, hi)
    if not plan.partial_writes:
        plan.pipeline = PipelineSpec(R, 1, {in_idx: esize * C, out_idx: esize * C}, set(), make)
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: RMS normalisation of whole rows
# --------------------------------------------------------------------------------------------------
def _match_rms_norm(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(rms_norm(load(x rows), load(gamma), eps))`` at the rows it was loaded from -> one fused row
    kernel per contiguous row range (python/asc/language/tile/unary_ops.py:225-237; the reference lowers to
    the Ascend C RmsNorm routine, lib/Conversion/LowerToAsc/LowerAscTile.cpp:190-289)."""
    value, out_t = eff.args
    node = _node(value, "rms_norm") if isinstance(value, Tile) else None
    if node is None:
        return None
    src, gamma, eps = node.args
    dtype = value.dtype
    if dtype not in (KT.float32, KT.float16) or out_t.dtype != dtype or gamma.dtype != dtype:
        raise _unsupported(f"rms_norm on {dtype} tiles (float32 and float16, one type throughout)")
    esize = dtype.bitwidth // 8
    fn_name = "asc_cuda_rms_norm_f32" if dtype == KT.float32 else "asc_cuda_rms_norm_f16"
    view = resolve_view(src) if _node(src, "load") or _is_materialised(src) else None
    gview = resolve_view(gamma) if _node(gamma, "load") else None
    if view is None or gview is None:
        if gview is not None and not _MATERIALISED and _matmul_leaves(src):
            return None        # a matmul result: _match_matmul_then_program writes it to a temporary and comes back
        raise _unsupported("rms_norm of tiles that are not loaded directly from global memory")
    if not eps.is_const:
        raise _unsupported("rms_norm with an epsilon that varies between blocks or iterations")
    if not _same_offsets(view.offsets, eff.attrs["offsets"]) or view.shape != value.shape:
        raise _unsupported("rms_norm stored at a different position than it was loaded from")
    if view.tensor.static_shape() != out_t.static_shape() or view.tensor.dtype != dtype or gview.tensor.dtype != dtype:
        raise _unsupported("rms_norm between tensors of different shapes or types")
    _check_fits(out_t)
    _check_fits(view.tensor)
    _check_fits(gview.tensor)
    R, C = _row_major_2d(out_t)
    tile_rows = 1 if len(value.shape) == 1 else value.shape[0]
    tile_cols = value.shape[-1]
    g_elems = 1
    for d in gamma.shape:
        g_elems *= d
    if gamma.shape[-1] != tile_cols or g_elems != tile_cols:
        raise _unsupported("rms_norm with a gamma tile that is not one row of the input's width")
    if tile_cols != C:
        # the mean runs over the tile's row; a window of a wider row would need a second pitch
        raise _unsupported("rms_norm of tiles narrower or wider than the tensor row")
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    row_off = PlainValue.const(0) if len(value.shape) == 1 else view.offsets[0]
    col_off = view.offsets[-1]
    r0 = eval_int(row_off, env, n)
    c0 = eval_int(col_off, env, n)
    if len(value.shape) == 1:       # a 1-D tensor of C elements is one row
        r0 = c0 // max(C, 1)
        c0 = c0 % max(C, 1)
    if n and (r0.min() < 0 or c0.min() < 0):
        raise RuntimeError("Negative tile offset in kernel")
    if n and c0.max() != 0:
        raise _unsupported("rms_norm tiles that do not start at the beginning of a row")
    g_off = np.zeros(n, dtype=np.int64)
    g_cols = gview.tensor.static_shape()[-1]
    for d, off in enumerate(gview.offsets):
        o = eval_int(off, env, n)
        if d < len(gview.offsets) - 1:
            o = o * g_cols       # gamma held as a [1, C] (or [k, C]) tensor
            if len(gview.offsets) > 2:
                raise _unsupported("rms_norm with gamma loaded from a tensor of rank above 2")
        g_off += o
    if n and (g_off.min() < 0 or not np.all(g_off == g_off[0])):
        raise _unsupported("rms_norm with gamma loaded from varying positions")
    gamma_off = int(g_off[0]) if n else 0
    if gamma_off + tile_cols > gview.tensor.base.numel:
        raise _unsupported("rms_norm with a gamma tile reaching past its tensor (zero padding)")
    intervals = merge_intervals(r0, np.minimum(r0 + tile_rows, R))
    if len(intervals) > MAX_CALLS:
        raise _unsupported("rms_norm kernel touching more than 4096 disjoint row ranges")
    plan = Plan("rms_norm")
    in_idx, out_idx, g_idx = view.tensor.base.index, out_t.base.index, gview.tensor.base.index
    plan.reads.update((in_idx, g_idx))
    plan.writes.add(out_idx)
    if not (intervals == [(0, R)] and R * C == out_t.base.numel):
        plan.partial_writes.add(out_idx)
    epsilon = float(eps.value)

    def make(lo: int, hi: int) -> List[Step]:
        def build(ptrs, stream, lo=lo, hi=hi):
            byte_off = esize * lo * C
            return (_p(ptrs[in_idx] + byte_off), _p(ptrs[g_idx] + esize * gamma_off), _p(ptrs[out_idx] + byte_off),
                    ctypes.c_int64(hi - lo), ctypes.c_int64(C), ctypes.c_int64(C), ctypes.c_float(epsilon), stream)
        return [Step(fn_name, build, f"rows [{lo}, {hi}) x {C} cols")]

    for lo, hi in intervals:
        plan.steps += make(lo, hi)
    if not plan.partial_writes and g_idx not in (in_idx, out_idx):
        plan.pipeline = PipelineSpec(R, 1, {in_idx: esize * C, out_idx: esize * C}, {g_idx}, make)
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: matmul (+ K loop with matmul_acc) with a fused store epilogue
# --------------------------------------------------------------------------------------------------
class _Epilogue:
    relu = False
    out_dtype: Optional[DataType] = None
    row_scale: Optional[GmView] = None   # int8 dequant: per-row scale vector
    col_scale: Optional[GmView] = None   # int8 dequant: per-column scale vector
    bias: Optional[GmView] = None        # one loaded row added to every row of the product before the ReLU


def _peel_identity_copies(tile: Tile) -> Tile:
    """Skip copies that keep shape and start at offset 0 (L0C -> L1 -> L0A round trips)."""
    while isinstance(tile, Tile) and tile.node.kind == "copy":
        node = tile.node
        src = node.args[0]
        if node.attrs["shape"] != src.shape or not all(o.is_const and o.value == 0 for o in node.attrs["offsets"]):
            break
        tile = src
    return tile


def _scale_vector(tile: Any, full_shape: Tuple[int, int]) -> Optional[Tuple[str, GmView]]:
    """``tile`` is a 1-D load broadcast along rows or columns of ``full_shape``: ("row"|"col", view)."""
    b = _node(tile, "broadcast")
    if b is None or tile.shape != full_shape:
        return None
    src = b.args[0]
    if not isinstance(src, Tile) or len(src.shape) != 2:
        return None
    kind = "row" if src.shape == (full_shape[0], 1) else "col" if src.shape == (1, full_shape[1]) else None
    if kind is None:
        return None
    while isinstance(src, Tile) and src.node.kind == "reshape":
        src = src.node.args[0]
    view = resolve_view(src) if _node(src, "load") else None
    if view is None or len(view.shape) != 1 or view.tensor.dtype != KT.float32:
        return None
    return kind, view


def _bias_row(tile: Any, full_shape: Tuple[int, int]) -> Optional[GmView]:
    """``tile`` is one loaded row (fp32, or fp16 / bf16 cast to fp32) broadcast over the rows of ``full_shape``."""
    b = _node(tile, "broadcast")
    if b is None or tile.shape != full_shape or tile.dtype != KT.float32:
        return None
    src = b.args[0]
    if not isinstance(src, Tile) or src.shape != (1, full_shape[1]):
        return None
    casts = 0
    while isinstance(src, Tile) and src.node.kind in ("reshape", "cast"):
        casts += src.node.kind == "cast"
        src = src.node.args[0]
    view = resolve_view(src) if _node(src, "load") else None
    if view is None or casts > 1 or view.tensor.dtype.name not in _OUT_CODE or not _is_zero_pad(view):
        return None
    if tuple(view.shape) not in ((full_shape[1],), (1, full_shape[1])) or len(view.tensor.static_shape()) != len(view.shape):
        return None
    return view


def _strip_epilogue(value: Tile) -> Tuple[Tile, _Epilogue]:
    epi = _Epilogue()
    epi.out_dtype = value.dtype
    v = value
    for _ in range(3):  # cast and relu in either order
        c = _node(v, "cast")
        if c is not None:
            v = c.args[0]
            continue
        r = _node(v, "unary", op="relu")
        if r is not None:
            epi.relu = True
            v = r.args[0]
            continue
        break
    # a bias row on the fp32 product: (a @ b) + row or row + (a @ b)
    add = _node(v, "binary", op="add")
    if add is not None and v.dtype == KT.float32 and len(v.shape) == 2:
        for core, other in ((add.args[0], add.args[1]), (add.args[1], add.args[0])):
            row = _bias_row(other, v.shape)
            if row is not None and isinstance(core, Tile) and core.node.kind in ("matmul", "acc"):
                epi.bias = row
                return core, epi
    # int8 dequantisation: cast_f32(acc) * row_scale * col_scale (either order)
    m1 = _node(v, "binary", op="mul")
    if m1 is not None and v.dtype == KT.float32 and len(v.shape) == 2:
        found = {}
        inner = None
        lhs, rhs = m1.args
        for first, second in ((lhs, rhs), (rhs, lhs)):
            sv = _scale_vector(second, v.shape)
            m2 = _node(first, "binary", op="mul")
            if sv is None or m2 is None:
                continue
            for core, other in ((m2.args[0], m2.args[1]), (m2.args[1], m2.args[0])):
                sv2 = _scale_vector(other, v.shape)
                c = _node(core, "cast")
                if sv2 is not None and c is not None and c.args[0].dtype == KT.int32 and sv2[0] != sv[0]:
                    found = {sv[0]: sv[1], sv2[0]: sv2[1]}
                    inner = c.args[0]
                    outer_is_col = sv[0] == "col"
            if inner is not None:
                break
        if inner is not None and outer_is_col:
            # (the fused epilogue computes (acc * a_scale[row]) * b_scale[col]; written the other way round the
            # product rounds differently, and the expression is left to the general path: the int32 product in a
            # temporary, then an elementwise program that multiplies in the order the kernel wrote)
            epi.row_scale, epi.col_scale = found["row"], found["col"]
            v = inner
    return v, epi


def _product_terms(node: Node, store_loops: Tuple[Loop, ...]) -> Optional[List[Tuple[Tile, Tile, bool, Tuple[Loop, ...]]]]:
    if node.kind == "matmul":
        return [(node.args[0], node.args[1], node.attrs["trans_b"], ())]
    if node.kind == "zeros_acc":
        return []
    if node.kind == "acc":
        prev, a, b = node.args
        head = _product_terms(prev, store_loops)
        if head is None:
            return None
        red = tuple(l for l in node.loops if l not in store_loops)
        return head + [(a, b, False, red)]
    return None


class _Window:
    """Rows x cols window of a 2-D row-major tensor with symbolic row/col offsets."""

    def __init__(self, tensor: Tensor, row: PlainValue, col: PlainValue, rows: int, cols: int):
        self.tensor, self.row, self.col, self.rows, self.cols = tensor, row, col, rows, cols


def _fake_tensor(key: str, shape: Tuple[int, int], dtype: DataType) -> Tensor:
    from ..language.core.ir_value import GlobalAddress
    base = GlobalAddress(key, dtype, key, shape[0] * shape[1])  # type: ignore[arg-type]
    return Tensor(base, tuple(PlainValue.const(d) for d in shape))


def _materialise_operand(trace: KernelTrace, tile: Tile, plan: Plan) -> Optional[_Window]:
    """A matmul operand computed elementwise from loaded tiles (a cast, an activation, a mask applied on the way
    from global memory to the cube unit): one program writes it, over every block and iteration that loads it, into
    a temporary laid out like the tensor its tile was loaded from; the product then reads the temporary there."""
    anchor = next((n for n in _loads_of(tile) if tuple(n.attrs["shape"]) == tile.shape and len(tile.shape) == 2
                   and len(n.args[0].static_shape()) == 2), None)
    if anchor is None:
        return None
    source = anchor.args[0]
    key = f"tmp{len(plan.temps)}"
    tmp = _fake_tensor(key, source.static_shape(), tile.dtype)
    offsets = anchor.attrs["offsets"]
    sub = _match_eltwise_program(trace, Effect("store", (tile, tmp), {"offsets": offsets}, tile.node.loops))
    if sub is None:
        return None
    plan.temps[key] = source.static_shape()[0] * source.static_shape()[1] * tile.dtype.sizeof()
    plan.temps.update(sub.temps)
    plan.steps.extend(sub.steps)
    plan.reads.update(r for r in sub.reads if r != key)
    return _Window(tmp, offsets[0], offsets[1], tile.shape[0], tile.shape[1])


def _operand_window(trace: KernelTrace, tile: Tile, plan: Plan) -> _Window:
    tile = _peel_identity_copies(tile)
    view = resolve_view(tile)
    if view is not None:
        if len(view.shape) != 2 or len(view.tensor.static_shape()) != 2:
            raise _unsupported("matmul operand that is not a 2-D tile of a 2-D tensor")
        if not _is_zero_pad(view):
            raise _unsupported("matmul operand loaded with a non-zero pad value")
        _check_fits(view.tensor)
        plan.reads.add(view.tensor.base.index)
        return _Window(view.tensor, view.offsets[0], view.offsets[1], view.shape[0], view.shape[1])
    if not _matmul_leaves(tile):
        w = _materialise_operand(trace, tile, plan)
        if w is None:
            raise _unsupported(f"matmul operand produced by '{tile.node.kind}'")
        return w
    # an operand computed on chip (chained matmul): materialise it in a temporary device buffer
    key = f"tmp{len(plan.temps)}"
    tmp = _fake_tensor(key, tile.shape, tile.dtype)
    plan.temps[key] = tile.size * tile.dtype.sizeof()
    zero = (PlainValue.const(0), PlainValue.const(0))
    if not _plan_matmul_value(trace, tile, tmp, zero, (), plan):
        raise _unsupported(f"matmul operand produced by '{tile.node.kind}'")
    return _Window(tmp, zero[0], zero[1], tile.shape[0], tile.shape[1])


def _merge_k_loop(a: _Window, b: _Window, red: Tuple[Loop, ...]) -> Tuple[_Window, _Window]:
    """Fold a K loop ``for k: acc += A[:, f(k):f(k)+kt] @ B[f(k):f(k)+kt, :]`` into one product."""
    if not red:
        return a, b
    if len(red) != 1:
        raise _unsupported("matmul_acc inside more than one reduction loop")
    loop = red[0]
    if not (loop.start.is_const and loop.stop.is_const and loop.step.is_const):
        raise _unsupported("K loop with run-time bounds")
    ks = np.arange(int(loop.start.value), int(loop.stop.value), int(loop.step.value), dtype=np.int64)
    if ks.size == 0:
        raise _unsupported("empty K loop")
    name = loop.name
    if name in a.row.symbols() or name in b.col.symbols():
        raise _unsupported("matmul_acc whose M or N offset changes inside the K loop")
    if not a.col.symbols() <= {name} or not b.row.symbols() <= {name}:
        raise _unsupported("K offset that depends on the block or an outer loop")
    ak = np.sort(eval_int(a.col, {name: ks}, ks.size))
    bk = np.sort(eval_int(b.row, {name: ks}, ks.size))
    kt = a.cols
    if b.rows != kt or not np.array_equal(ak, bk) or not np.array_equal(ak, ak[0] + kt * np.arange(ks.size)):
        raise _unsupported("K loop whose slices do not tile the K dimension contiguously")
    k_lo, k_tot = int(ak[0]), int(kt * ks.size)
    return (_Window(a.tensor, a.row, PlainValue.const(k_lo), a.rows, k_tot),
            _Window(b.tensor, PlainValue.const(k_lo), b.col, k_tot, b.cols))


def _plan_matmul_value(trace: KernelTrace, value: Tile, out_t: Tensor, out_offsets: Sequence[PlainValue],
                       loops: Tuple[Loop, ...], plan: Plan, guards: Tuple = ()) -> bool:
    """Append the steps computing ``value`` (a matmul with epilogue) into ``out_t`` at ``out_offsets``.
    Returns False when ``value`` is not a matmul expression."""
    if not isinstance(value, Tile) or len(value.shape) != 2:
        return False
    core, epi = _strip_epilogue(value)
    terms = _product_terms(core.node, loops) if isinstance(core, Tile) else None
    if terms is None:
        return False
    if len(terms) != 1:
        raise _unsupported(f"accumulator fed by {len(terms)} matmul_acc calls (exactly one is supported)")
    a_tile, b_tile, trans_b, red = terms[0]
    if trans_b:
        raise _unsupported("matmul with trans_b outside the attention pattern")
    a_w, b_w = _merge_k_loop(_operand_window(trace, a_tile, plan), _operand_window(trace, b_tile, plan), red)
    in_dtype = a_w.tensor.dtype
    if b_w.tensor.dtype != in_dtype:
        raise _unsupported("matmul operands of different types")
    if len(out_t.static_shape()) != 2:
        raise _unsupported("matmul result stored to a tensor that is not 2-D")
    if epi.out_dtype != out_t.dtype:
        raise _unsupported(f"storing a {epi.out_dtype} tile into a {out_t.dtype} tensor")
    if (epi.row_scale is None) != (in_dtype != KT.int8 or epi.out_dtype == KT.int32):
        raise _unsupported("int8 matmul must be stored as int32 or dequantised with row and column scales")
    _check_fits(out_t)
    mt, nt = value.shape
    a_rows, a_cols = a_w.tensor.static_shape()
    b_rows, b_cols = b_w.tensor.static_shape()
    c_rows, c_cols = out_t.static_shape()

    env = enumerate_instances(trace.core_num, loops, guards)
    n = env_count(env)
    ro, co = eval_int(out_offsets[0], env, n), eval_int(out_offsets[1], env, n)
    ar, ak = eval_int(a_w.row, env, n), eval_int(a_w.col, env, n)
    bk, bc = eval_int(b_w.row, env, n), eval_int(b_w.col, env, n)
    cols = [ro, co, ar, ak, bk, bc]
    if epi.row_scale is not None:
        cols += [eval_int(epi.row_scale.offsets[0], env, n), eval_int(epi.col_scale.offsets[0], env, n)]
    if epi.bias is not None:
        if in_dtype.name not in _DTYPE_CODE_16:
            raise _unsupported(f"bias row in the epilogue of a {in_dtype} matmul")
        _check_fits(epi.bias.tensor)
        bias_ld = epi.bias.tensor.static_shape()[-1]
        bias_col = eval_int(epi.bias.offsets[-1], env, n)
        bias_row = eval_int(epi.bias.offsets[0], env, n) if len(epi.bias.offsets) == 2 else np.zeros(n, dtype=np.int64)
        cols += [bias_row, bias_col]
    inst = np.unique(np.stack(cols, axis=1), axis=0)   # identical instances (e.g. every block) collapse
    if inst.size and inst.min() < 0:
        raise RuntimeError("Negative tile offset in kernel")
    ro, co, ar, ak, bk, bc = (inst[:, i] for i in range(6))
    # (A's K range starts at column ak, B's at row bk: equal when both index one K axis, different when B is a stack
    # of matrices, as in a loop over a batch)
    if epi.row_scale is not None and (np.any(inst[:, 6] != ar) or np.any(inst[:, 7] != bc)
                                      or epi.row_scale.shape[0] != mt or epi.col_scale.shape[0] != nt):
        raise _unsupported("dequantisation scales that are not indexed by the tile's rows / columns")
    bias_at = np.zeros(inst.shape[0], dtype=np.int64)     # element offset of each tile's first bias value
    if epi.bias is not None:
        rows_of_bias = epi.bias.tensor.static_shape()[0] if len(epi.bias.offsets) == 2 else 1
        if np.any(inst[:, 6] >= rows_of_bias) or np.any(inst[:, 7] + np.minimum(nt, c_cols - co) > bias_ld):
            raise _unsupported("bias row that reaches past the end of its tensor (zero padding)")
        bias_at = inst[:, 6] * bias_ld + inst[:, 7]
    k_eff = np.minimum(np.minimum(a_w.cols, a_cols - ak), b_rows - bk)
    m_eff = np.minimum(mt, c_rows - ro)
    n_eff = np.minimum(nt, c_cols - co)
    if np.any(k_eff <= 0):
        raise _unsupported("matmul tile outside the K extent of its operands")
    if np.any(a_rows - ar < m_eff) or np.any(b_cols - bc < n_eff):
        raise _unsupported("matmul tile that reads padded rows of A or padded columns of B")
    keep = (m_eff > 0) & (n_eff > 0)

    # one call when the tiles form a full grid over a rectangle, else one call per tile
    calls: List[Tuple[int, ...]] = []   # (ro, co, ar, bc, k0, M, N, K)
    ru, cu = np.unique(ro[keep]), np.unique(co[keep])
    grid_ok = (keep.all() and inst.shape[0] == ru.size * cu.size and np.all(ak == ak[0]) and np.all(bk == bk[0]) and
               np.all(k_eff == k_eff[0]) and np.all(ar - ro == ar[0] - ro[0]) and np.all(bc - co == bc[0] - co[0]) and
               (epi.bias is None or np.all(bias_at - co == bias_at[0] - co[0])) and
               np.array_equal(ru, ru[0] + mt * np.arange(ru.size)) and
               np.array_equal(cu, cu[0] + nt * np.arange(cu.size)) and
               np.unique(np.stack([ro, co], axis=1), axis=0).shape[0] == inst.shape[0])
    if inst.shape[0] and grid_ok:
        M = int(min(ru[-1] + mt, c_rows) - ru[0])
        N = int(min(cu[-1] + nt, c_cols) - cu[0])
        calls.append((int(ru[0]), int(cu[0]), int(ru[0] + ar[0] - ro[0]), int(cu[0] + bc[0] - co[0]), int(ak[0]),
                      M, N, int(k_eff[0]), int(bk[0]), int(cu[0] + bias_at[0] - co[0])))
    else:
        for i in np.nonzero(keep)[0]:
            calls.append((int(ro[i]), int(co[i]), int(ar[i]), int(bc[i]), int(ak[i]), int(m_eff[i]), int(n_eff[i]),
                          int(k_eff[i]), int(bk[i]), int(bias_at[i])))
        if len(calls) > MAX_CALLS:
            raise _unsupported("matmul kernel whose tiles do not form a grid and exceed 4096 calls")
        if calls:
            c = np.array(calls, dtype=np.int64)
            rect = np.stack([c[:, 0], c[:, 0] + c[:, 5], c[:, 1], c[:, 1] + c[:, 6]], axis=1)
            clash = _rects_overlap(rect, rect)
            np.fill_diagonal(clash, False)
            if clash.any():
                raise _unsupported("matmul tiles computed from different operands that overlap in the output "
                                   "(the last writer would win)")

    a_idx, b_idx, c_idx = a_w.tensor.base.index, b_w.tensor.base.index, out_t.base.index
    if c_idx in (a_idx, b_idx):
        # (tiles of the product run concurrently: one would overwrite operand rows or columns another still reads)
        raise _unsupported("matmul stored into one of its own operands")
    plan.writes.add(c_idx)
    if not (len(calls) == 1 and calls[0][0] == 0 and calls[0][1] == 0 and calls[0][5] == c_rows and
            calls[0][6] == c_cols and c_rows * c_cols == out_t.base.numel):
        plan.partial_writes.add(c_idx)
    es = in_dtype.sizeof()
    osz = out_t.dtype.sizeof()
    lda, ldb, ldc = a_cols, b_cols, c_cols
    flags = 1 if epi.relu else 0
    sa_idx = sb_idx = bias_idx = None
    if epi.bias is not None:
        bias_idx, bias_code = epi.bias.tensor.base.index, _OUT_CODE[epi.bias.tensor.dtype.name]
        bias_size = epi.bias.tensor.dtype.sizeof()
        if bias_idx == out_t.base.index:
            raise _unsupported("bias row loaded from the tensor the product is stored to")
        plan.reads.add(bias_idx)
    if in_dtype == KT.int8:
        if epi.relu:
            raise _unsupported("ReLU on an int8 matmul")
        if epi.row_scale is not None:
            if out_t.dtype != KT.float16:
                raise _unsupported("dequantised int8 matmul must be stored as float16")
            sa_idx, sb_idx = epi.row_scale.tensor.base.index, epi.col_scale.tensor.base.index
            plan.reads.update((sa_idx, sb_idx))
    elif in_dtype == KT.float32 or in_dtype.name in _DTYPE_CODE_16:
        if out_t.dtype.name not in _OUT_CODE:
            raise _unsupported(f"matmul result type {out_t.dtype}")
    else:
        raise _unsupported(f"matmul on {in_dtype} operands")

    def gemm_step(r0: int, c0: int, a0: int, b0: int, k0: int, M: int, N: int, K: int, kb: Optional[int] = None,
                  bias0: int = 0) -> Step:
        kb = k0 if kb is None else kb         # first row of B's K range
        a_off, b_off, c_off = (a0 * lda + k0) * es, (kb * ldb + b0) * es, (r0 * ldc + c0) * osz
        dims = (ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(lda), ctypes.c_int64(ldb),
                ctypes.c_int64(ldc))
        note = f"C[{r0}:{r0 + M}, {c0}:{c0 + N}] = A[{a0}:, {k0}:{k0 + K}] @ B[{kb}:, {b0}:]"
        if in_dtype == KT.int8:
            if sa_idx is not None:
                def build(ptrs, stream):
                    return (_p(ptrs[a_idx] + a_off), _p(ptrs[b_idx] + b_off), None, _p(ptrs[c_idx] + c_off),
                            _p(ptrs[sa_idx] + 4 * a0), _p(ptrs[sb_idx] + 4 * b0), *dims, stream)
            else:
                def build(ptrs, stream):
                    return (_p(ptrs[a_idx] + a_off), _p(ptrs[b_idx] + b_off), _p(ptrs[c_idx] + c_off), None, None,
                            None, *dims, stream)
            return Step("asc_cuda_gemm_i8", build, note)
        oc = _OUT_CODE[out_t.dtype.name]
        if in_dtype == KT.float32:
            def build(ptrs, stream):
                return (_p(ptrs[a_idx] + a_off), _p(ptrs[b_idx] + b_off), _p(ptrs[c_idx] + c_off), *dims,
                        ctypes.c_int32(oc), ctypes.c_int32(flags), stream)
            return Step("asc_cuda_gemm_f32", build, note)
        ic = _DTYPE_CODE_16[in_dtype.name]
        if bias_idx is not None:
            def build(ptrs, stream):
                return (_p(ptrs[a_idx] + a_off), _p(ptrs[b_idx] + b_off), _p(ptrs[c_idx] + c_off),
                        _p(ptrs[bias_idx] + bias0 * bias_size), *dims, ctypes.c_int32(ic), ctypes.c_int32(oc),
                        ctypes.c_int32(bias_code), ctypes.c_int32(flags), stream)
            return Step("asc_cuda_gemm_f16_bias", build, note + f" + bias[{bias0}:{bias0 + N}]")

        def build(ptrs, stream):
            return (_p(ptrs[a_idx] + a_off), _p(ptrs[b_idx] + b_off), _p(ptrs[c_idx] + c_off), *dims,
                    ctypes.c_int32(ic), ctypes.c_int32(oc), ctypes.c_int32(flags), stream)
        return Step("asc_cuda_gemm_f16", build, note)

    for call in calls:
        plan.steps.append(gemm_step(*call))
    # one full-output call whose operands are plain global tensors: rows of A and C can be streamed
    if (len(calls) == 1 and c_idx not in plan.partial_writes and calls[0][2] == 0 and calls[0][3] == 0 and
            calls[0][4] == 0 and calls[0][8] == 0 and all(isinstance(i, int) for i in (a_idx, b_idx, c_idx)) and
            len({a_idx, b_idx, c_idx}) == 3 and in_dtype != KT.float32 and
            (bias_idx is None or (isinstance(bias_idx, int) and bias_idx not in (a_idx, c_idx)))):
        _, _, _, _, _, M, N, K, _, bias_first = calls[0]
        streamed = {a_idx: lda * es, c_idx: ldc * osz}
        resident = {b_idx}
        if sa_idx is not None:
            streamed[sa_idx] = 4
            resident.add(sb_idx)
        if bias_idx is not None:
            resident.add(bias_idx)
        plan.pipeline = PipelineSpec(M, 256, streamed, resident,
                                     lambda lo, hi: [gemm_step(lo, 0, lo, 0, 0, hi - lo, N, K, None, bias_first)])
    return True


def _match_matmul(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    value, out_t = eff.args
    plan = Plan("matmul")
    try:
        if not _plan_matmul_value(trace, value, out_t, eff.attrs["offsets"], eff.loops, plan, eff.guards):
            return None
    except NotImplementedError as refusal:
        # an epilogue the GEMM kernels do not fuse (an int8 product cast to fp32, a ReLU on one, ...): the general
        # path computes the bare product into a temporary and finishes the expression with a program
        if isinstance(value, Tile) and value.node.kind not in ("matmul", "acc"):
            try:
                alt = _match_matmul_then_program(trace, eff)
            except NotImplementedError:
                alt = None
            if alt is not None:
                return alt
        raise refusal
    return plan


def _match_copy(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(load(...))`` of a tile whose element type the elementwise kernels do not compute on (8-bit and 64-bit
    types): a move of bytes, window by window (``asc_cuda_copy_2d``).  Types the programs know keep their path."""
    value, out_t = eff.args
    if eff.kind != "store" or not isinstance(value, Tile) or value.dtype.name in _ELT_TYPE or value.dtype != out_t.dtype:
        return None
    view = resolve_view(value) if value.node.kind in ("load", "copy") else None
    if view is None or view.tensor.dtype != value.dtype or tuple(view.shape) != tuple(value.shape):
        return None
    _check_fits(out_t)
    _check_fits(view.tensor)
    offsets = eff.attrs["offsets"]
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    if n > MAX_CALLS:
        raise _unsupported("copy kernel with more than 4096 tiles")
    src_g = _Geometry(view.tensor, view.offsets, view.shape, False, env, n)      # refuses tiles past the end
    dst_g = _Geometry(out_t, offsets, value.shape, False, env, n)
    esize = value.dtype.sizeof()
    # the window one call moves: rows x cols elements with a pitch on either side
    if src_g.pitch is None and dst_g.pitch is None:
        rows, cols = 1, src_g.numel
    else:
        rows, cols = (src_g.rows, src_g.cols) if src_g.pitch is not None else (dst_g.rows, dst_g.cols)
        for g in (src_g, dst_g):
            if g.pitch is not None and (g.rows, g.cols) != (rows, cols):
                raise _unsupported("copy between windows of different shapes")
    src_ld = src_g.pitch if src_g.pitch is not None else cols
    dst_ld = dst_g.pitch if dst_g.pitch is not None else cols
    src_idx, dst_idx = view.tensor.base.index, out_t.base.index
    if src_idx == dst_idx:
        raise _unsupported("copy inside one tensor")
    pairs = sorted(set(zip(src_g.start.tolist(), dst_g.start.tolist())), key=lambda p: p[1])
    rect = _flat_rects(out_t.static_shape()[-1] if out_t.static_shape() else 1, np.array([p[1] for p in pairs], dtype=np.int64),
                       dst_g.numel, dst_g.rows, dst_g.cols, dst_g.pitch)
    clash = _rects_overlap(rect, rect)
    np.fill_diagonal(clash, False)
    if clash.any():
        raise _unsupported("copies of different tiles into overlapping ranges (the last writer would win)")
    calls: List[Tuple[int, int, int]] = []       # (first source element, first destination element, rows)
    for s0, d0 in pairs:
        if calls:
            ps, pd, prow = calls[-1]
            if s0 == ps + prow * src_ld and d0 == pd + prow * dst_ld:
                calls[-1] = (ps, pd, prow + rows)      # the next rows of the same two matrices
                continue
        calls.append((s0, d0, rows))
    plan = Plan("copy")
    plan.reads.add(src_idx)
    plan.writes.add(dst_idx)
    if not (len(calls) == 1 and calls[0][1] == 0 and dst_ld == cols and calls[0][2] * cols == out_t.base.numel):
        plan.partial_writes.add(dst_idx)

    def make_step(s0: int, d0: int, call_rows: int) -> Step:
        def build(ptrs, stream):
            return (_p(ptrs[dst_idx] + esize * d0), _p(ptrs[src_idx] + esize * s0), ctypes.c_int64(call_rows),
                    ctypes.c_int64(cols * esize), ctypes.c_int64(dst_ld * esize), ctypes.c_int64(src_ld * esize), stream)
        return Step("asc_cuda_copy_2d", build, f"[{call_rows}, {cols}] {value.dtype.name} from {s0} to {d0}")

    for call in calls:
        plan.steps.append(make_step(*call))
    return plan


def _column_reductions(value: Any, shape: Tuple[int, ...], limit: int = 4096) -> List[Tile]:
    """The reductions along the first axis of [rows, cols] tiles that the expression of ``value`` uses (through a
    ``broadcast_to(rows, cols)`` of a row computed from them), innermost first."""
    found: List[Tile] = []
    seen = set()

    def visit(v: Any) -> None:
        if len(seen) > limit:
            return
        if isinstance(v, Tile):
            if id(v.node) in seen:
                return
            seen.add(id(v.node))
            for a in v.node.args:
                visit(a)
            for a in v.node.attrs.values():
                if isinstance(a, (Tile, PlainValue)):
                    visit(a)
            if v.node.kind == "reduce" and v.node.attrs["dims"] == (0, ) and v.node.args[0].shape == shape:
                found.append(v)
        elif isinstance(v, PlainValue) and v.op not in ("const", "sym"):
            for a in v.args:
                if isinstance(a, (Tile, PlainValue)):
                    visit(a)
    visit(value)
    return found


def _match_column_statistics(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(f(x, reduce(g(x), 0, keep_dims=True).broadcast_to(rows, cols), ...))``: an elementwise expression that
    uses reductions of [rows, cols] tiles along their first axis, repeated over the rows (a softmax or a normalisation
    down the columns).  Every such reduction is computed first, innermost first, by a column program into a temporary
    matrix of the result's shape (the row of the tile's own window, so every tile has its own), and is then an
    ordinary broadcast-row operand of what follows; the last step is one elementwise program."""
    value, out_t = eff.args
    if eff.kind != "store" or not isinstance(value, Tile) or len(value.shape) != 2 or len(out_t.static_shape()) != 2:
        return None
    reductions = _column_reductions(value, value.shape)
    if not reductions or value.node.kind == "reduce":
        return None
    offsets = eff.attrs["offsets"]
    rows, cols = value.shape
    plan = Plan("column:statistics")
    try:
        for src in reductions:
            key = f"tmp{len(plan.temps)}"
            tmp = _fake_tensor(key, out_t.static_shape(), src.dtype)
            plan.temps[key] = out_t.base.numel * src.dtype.sizeof()
            row_tile = Tile((1, cols), src.dtype, src.node, src.location)           # the reduction, kept as one row
            sub_eff = Effect("store", (row_tile, tmp), {"offsets": offsets}, eff.loops, eff.guards)
            sub = _match_col_reduce(trace, sub_eff) or _match_reduce(trace, sub_eff)
            if sub is None:
                raise _unsupported("reduction along the first axis that no kernel computes")
            sub.reads.discard(key)
            plan.steps.extend(sub.steps)
            plan.reads.update(r for r in sub.reads if not (isinstance(r, str) and r.startswith("tmp")))
            _MATERIALISED[id(src.node)] = _Operand(tmp, offsets, (1, cols), bcast=True)
        tail = _match_eltwise_program(trace, eff)
    finally:
        _MATERIALISED.clear()
    if tail is None:
        raise _unsupported("expression around reductions along the first axis that is not elementwise")
    plan.temps.update(tail.temps)
    plan.steps.extend(tail.steps)
    plan.reads.update(r for r in tail.reads if not (isinstance(r, str) and r.startswith("tmp")))
    plan.writes.update(tail.writes)
    plan.partial_writes.update(tail.partial_writes)
    return plan


_MAX_PRODUCTS = 4      # matmul results one stored expression may combine (a temporary matrix each)


def _matmul_leaves(value: Any, limit: int = 4096) -> List[Tile]:
    """The matmul results (``matmul`` / ``matmul_acc`` accumulators) an expression is computed from."""
    found: List[Tile] = []
    seen = set()
    stack = [value]
    while stack and len(seen) < limit:
        v = stack.pop()
        if isinstance(v, Tile):
            if id(v.node) in seen:
                continue
            seen.add(id(v.node))
            if v.node.kind in ("matmul", "acc"):
                found.append(v)
                continue
            stack.extend(v.node.args)
            stack.extend(a for a in v.node.attrs.values() if isinstance(a, (Tile, PlainValue)))
        elif isinstance(v, PlainValue) and v.op not in ("const", "sym"):
            stack.extend(a for a in v.args if isinstance(a, (Tile, PlainValue)))
    return found


def _match_matmul_then_program(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    """``store(f(a @ b, other tiles...))`` with an elementwise ``f`` the matmul epilogues do not cover (a bias row,
    an activation, a residual): the product goes to a temporary matrix of the result's shape, then one elementwise
    program reads it back together with the other operands.  The reference fuses such an expression on chip between
    the cube unit's output buffer and the vector unit (MatmulOp + vector calls, lib/Conversion/LowerToAsc/
    LowerAscTile.cpp); here it costs one extra pass over the fp32 product."""
    value, out_t = eff.args
    if eff.kind != "store" or not isinstance(value, Tile) or len(value.shape) != 2 or value.node.kind in ("matmul", "acc"):
        return None
    leaves = _matmul_leaves(value)
    if not leaves:
        return None
    if len(leaves) > _MAX_PRODUCTS:
        raise _unsupported(f"expression that combines more than {_MAX_PRODUCTS} matmul results")
    if _value_from_deeper_loop(value, eff.loops, stop=tuple(id(mm.node) for mm in leaves)):
        return None          # something besides the accumulators is carried out of a loop
    if any(mm.shape != value.shape for mm in leaves) or len(out_t.static_shape()) != 2:
        raise _unsupported("matmul result reshaped or stored to a tensor that is not 2-D before its elementwise epilogue")
    offsets = eff.attrs["offsets"]
    plan = Plan("matmul+program")
    rows, cols = out_t.static_shape()
    keys = []
    try:
        for mm in leaves:
            key = f"tmp{len(plan.temps)}"
            tmp = _fake_tensor(key, (rows, cols), mm.dtype)
            plan.temps[key] = rows * cols * mm.dtype.sizeof()
            if not _plan_matmul_value(trace, mm, tmp, offsets, eff.loops, plan, eff.guards):
                return None
            keys.append(key)
            _MATERIALISED[id(mm.node)] = _Operand(tmp, offsets, mm.shape)
        # the rest of the expression reads the products like loaded tiles: a fused row kernel where one fits
        # (softmax, rms_norm of the product), else an elementwise or row program
        tail, refusal = None, None
        for finish in (_match_softmax, _match_rms_norm, _match_eltwise_program):
            try:
                tail = finish(trace, eff)
            except NotImplementedError as e:      # e.g. softmax of a scaled product: the row program takes it
                refusal = refusal or e
                continue
            if tail is not None:
                break
    finally:
        _MATERIALISED.clear()
    if tail is None:
        raise refusal or _unsupported("expression around a matmul result that is not elementwise")
    for key in keys:
        tail.reads.discard(key)
    plan.temps.update(tail.temps)
    plan.steps.extend(tail.steps)
    plan.reads.update(tail.reads)
    plan.writes.update(tail.writes)
    plan.partial_writes.update(tail.partial_writes)
    return plan


# --------------------------------------------------------------------------------------------------
# Pattern: attention forward, written per query tile as softmax(scale * Q K^T [+ causal mask]) V
# --------------------------------------------------------------------------------------------------
def _match_attention(trace: KernelTrace, eff: Effect) -> Optional[Plan]:
    value, out_t = eff.args
    if not isinstance(value, Tile) or len(value.shape) != 2:
        return None
    v = value
    c = _node(v, "cast")
    if c is not None:
        v = c.args[0]
    pv = _node(v, "matmul", trans_b=False)
    if pv is None:
        return None
    p_tile, v_tile = pv.args
    pc = _node(p_tile, "cast")
    sm = _node(pc.args[0] if pc is not None else p_tile, "softmax")
    if sm is None:
        return None
    s_tile = sm.args[0]
    causal = False
    q_off = kv_off = None
    cm = _node(s_tile, "causal_mask")
    if cm is not None:
        causal = True
        q_off, kv_off = cm.attrs["q_offset"], cm.attrs["kv_offset"]
        s_tile = cm.args[0]
    mul = _node(s_tile, "binary", op="mul")
    if mul is None:
        raise _unsupported("attention scores must be scaled as (q @ k^T) * scale")
    qk = scale = None
    for x, y in ((mul.args[0], mul.args[1]), (mul.args[1], mul.args[0])):
        if _node(x, "matmul", trans_b=True) is not None and isinstance(y, PlainValue) and y.is_const:
            qk, scale = x.node, float(y.value)
    if qk is None:
        raise _unsupported("attention scores must be asc2.matmul(q, k, trans_b=True) times a constant scale")
    q_tile, k_tile = qk.args
    views = [resolve_view(t) if _node(t, "load") else None for t in (q_tile, k_tile, v_tile)]
    if any(x is None for x in views):
        raise _unsupported("attention operands must be loaded directly from global memory")
    qv, kv, vv = views
    dt = qv.tensor.dtype
    if dt.name not in _DTYPE_CODE_16 or kv.tensor.dtype != dt or vv.tensor.dtype != dt or out_t.dtype != dt \
            or value.dtype != dt:
        raise _unsupported("attention needs float16 or bfloat16 Q, K, V and O of one type")
    for t in (qv.tensor, kv.tensor, vv.tensor, out_t):
        _check_fits(t)
        if len(t.static_shape()) != 2:
            raise _unsupported("attention tensors must be viewed as [batch*heads*seq, head_dim]")
    rows, D = out_t.static_shape()
    tq = qv.shape[0]
    S = kv.shape[0]
    if any(t.static_shape() != (rows, D) for t in (qv.tensor, kv.tensor, vv.tensor)):
        raise _unsupported("attention Q, K, V, O must have the same [rows, head_dim] shape")
    if qv.shape[1] != D or kv.shape != (S, D) or vv.shape != (S, D) or rows % S != 0 or S % tq != 0:
        raise _unsupported("attention tiles must span the head dimension, K/V tiles one whole sequence")
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    row0 = eval_int(eff.attrs["offsets"][0], env, n)
    checks = [
        np.array_equal(np.sort(row0), np.arange(0, rows, tq)),
        np.array_equal(eval_int(qv.offsets[0], env, n), row0),
        np.array_equal(eval_int(kv.offsets[0], env, n), (row0 // S) * S),
        np.array_equal(eval_int(vv.offsets[0], env, n), (row0 // S) * S),
        all(not np.any(eval_int(x.offsets[1], env, n)) for x in (qv, kv, vv)),
        not np.any(eval_int(eff.attrs["offsets"][1], env, n)),
    ]
    if causal:
        checks.append(np.array_equal(eval_int(q_off, env, n), row0 % S))
        checks.append(not np.any(eval_int(kv_off, env, n)))
    if not all(checks):
        raise _unsupported("attention kernel whose tiles do not cover every query tile of every head exactly once")
    plan = Plan("attention")
    idx = [t.base.index for t in (qv.tensor, kv.tensor, vv.tensor, out_t)]
    if idx[3] in idx[1:3]:
        # (every query tile reads all keys and values of its head while other tiles already store their results)
        raise _unsupported("attention stored into its own K or V tensor")
    plan.reads.update(idx[:3])
    plan.writes.add(idx[3])
    if rows * D != out_t.base.numel:
        plan.partial_writes.add(idx[3])
    heads = rows // S

    head_bytes = S * D * 2

    def make(lo: int, hi: int) -> List[Step]:
        def build(ptrs, stream, lo=lo, hi=hi):
            off = lo * head_bytes
            return (_p(ptrs[idx[0]] + off), _p(ptrs[idx[1]] + off), _p(ptrs[idx[2]] + off), _p(ptrs[idx[3]] + off),
                    ctypes.c_int32(hi - lo), ctypes.c_int32(1), ctypes.c_int32(S), ctypes.c_int32(D),
                    ctypes.c_float(scale), ctypes.c_int32(int(causal)), ctypes.c_int32(_DTYPE_CODE_16[dt.name]),
                    stream)
        return [Step("asc_cuda_attn_fwd_f16", build, f"{hi - lo} heads x {S} x {D}, causal={causal}")]

    plan.steps += make(0, heads)
    if not plan.partial_writes and len(set(idx)) == 4:
        plan.pipeline = PipelineSpec(heads, 1, {i: head_bytes for i in idx}, set(), make)
    return plan


# --------------------------------------------------------------------------------------------------
# Write-after-write order: footprints of stores and the order the plan applies them in
# --------------------------------------------------------------------------------------------------
def _rects_overlap(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Pairwise overlap of two sets of rectangles ``[row_lo, row_hi, col_lo, col_hi)``: a bool matrix [len(a), len(b)]."""
    return ((a[:, None, 0] < b[None, :, 1]) & (b[None, :, 0] < a[:, None, 1]) &
            (a[:, None, 2] < b[None, :, 3]) & (b[None, :, 2] < a[:, None, 3]))


def _flat_rects(width: int, start: np.ndarray, numel: int, rows: int = 1, cols: int = 0,
                pitch: Optional[int] = None) -> np.ndarray:
    """Rectangles over a tensor seen as rows of ``width`` elements for windows that begin at flat index ``start``:
    ``rows`` x ``cols`` with a row pitch, or one contiguous range of ``numel`` elements.  A range that spans several
    rows is widened to whole rows (conservative)."""
    width = max(1, width)
    r0, c0 = start // width, start % width
    if pitch is not None:
        return np.stack([r0, r0 + rows, c0, c0 + cols], axis=1)
    one_row = c0 + numel <= width
    r1 = np.where(one_row, r0 + 1, -((-(start + numel)) // width))
    return np.stack([r0, r1, np.where(one_row, c0, 0), np.where(one_row, c0 + numel, width)], axis=1)


MAX_ORDER_PAIRS = 1 << 24    # instance pairs the write-order checks compare exactly


def _store_footprint(trace: KernelTrace, eff: Effect):
    """``(env, rects)`` of a store or atomic effect: the symbol bindings of its instances and the rectangle of the
    output tensor (rows of its last dimension) each instance writes, clipped to the tensor."""
    value, out_t = eff.args
    offsets = eff.attrs["offsets"]
    tshape = out_t.static_shape()
    width = tshape[-1] if tshape else 1
    env = enumerate_instances(trace.core_num, eff.loops, eff.guards)
    n = env_count(env)
    shape = value.shape if isinstance(value, Tile) and eff.kind != "store_scalar" else None
    if shape is None:
        start = eval_int(_flat_scalar_offset(tshape, offsets), env, n)
        return env, _flat_rects(width, start, 1)
    window = _flat_window(out_t, offsets, shape)
    if window is not None:
        start = eval_int(window[0], env, n)
        total = 1
        for d in tshape:
            total *= d
        rects = _flat_rects(width, start, window[1])
        rects[:, 1] = np.minimum(rects[:, 1], -(-total // max(1, width)))
        return env, rects
    if len(tshape) == 2 and len(shape) == 2:
        r0, c0 = eval_int(offsets[0], env, n), eval_int(offsets[1], env, n)
        return env, np.stack([r0, np.minimum(r0 + shape[0], tshape[0]), c0, np.minimum(c0 + shape[1], tshape[1])], axis=1)
    return env, None


def _check_effect_order(trace: KernelTrace, first: Effect, second: Effect, cache: Dict[int, Any]) -> None:
    """The plan applies ``first`` over all blocks and iterations, then ``second``.  Inside one block the kernel
    instead interleaves them iteration by iteration: if an instance of ``first`` that runs *after* an instance of
    ``second`` (a later iteration of a loop both are in) writes elements that instance also writes, the kernel
    leaves ``first``'s data there and the plan would leave ``second``'s.  Such kernels are refused."""
    if first.kind == "atomic" and second.kind == "atomic" and first.attrs.get("kind") == second.attrs.get("kind"):
        return                      # accumulations of one kind commute
    shared = 0
    while shared < min(len(first.loops), len(second.loops)) and first.loops[shared] is second.loops[shared]:
        shared += 1
    if shared == 0:
        return                      # `first` is complete in every block before `second` starts
    for e in (first, second):
        if id(e) not in cache:
            cache[id(e)] = _store_footprint(trace, e)
    (env_a, ra), (env_b, rb) = cache[id(first)], cache[id(second)]
    refuse = _unsupported(f"kernel '{trace.fn_name}' overwrites, in a later loop iteration, elements that another store "
                          "of an earlier iteration wrote after it in program order")
    if ra is None or rb is None or ra.shape[0] * rb.shape[0] > MAX_ORDER_PAIRS:
        # too many instances to compare pair by pair: any overlap of the two footprints is refused
        if ra is None or rb is None:
            raise refuse
        width = max(int(ra[:, 3].max(initial=1)), int(rb[:, 3].max(initial=1)))
        ia = merge_intervals(ra[:, 0] * width + ra[:, 2], (ra[:, 1] - 1) * width + ra[:, 3])
        ib = merge_intervals(rb[:, 0] * width + rb[:, 2], (rb[:, 1] - 1) * width + rb[:, 3])
        j = 0
        for lo, hi in ia:
            while j < len(ib) and ib[j][1] <= lo:
                j += 1
            if j < len(ib) and ib[j][0] < hi:
                raise refuse
        return
    names = ["block_idx"] + [l.name for l in first.loops[:shared]]
    later = np.zeros((ra.shape[0], rb.shape[0]), dtype=bool)      # `first`'s instance runs after `second`'s
    equal = np.ones_like(later)
    for k, name in enumerate(names):
        a, b = env_a[name][:, None], env_b[name][None, :]
        if k == 0:
            equal &= a == b         # only instances of one block are ordered
            continue
        later |= equal & (a > b)
        equal &= a == b
    if np.any(later & _rects_overlap(ra, rb)):
        raise refuse


# --------------------------------------------------------------------------------------------------
# Entry point
# --------------------------------------------------------------------------------------------------
_MATCHERS = (_match_attention, _match_softmax, _match_rms_norm, _match_elementwise, _match_matmul,
             _match_matmul_then_program, _match_column_statistics, _match_eltwise_program, _match_copy,
             _match_row_result, _match_row_scalar, _match_col_reduce, _match_reduce)


def _is_identity_store(eff: Effect) -> bool:
    value, out_t = eff.args
    view = resolve_view(value) if _node(value, "load") else None
    return (view is not None and view.tensor.base.index == out_t.base.index and view.shape == value.shape
            and view.tensor.static_shape() == out_t.static_shape() and _same_offsets(view.offsets, eff.attrs["offsets"]))


def _value_from_deeper_loop(value: Any, loops: Tuple[Loop, ...], stop: Tuple[int, ...] = ()) -> bool:
    """True when the stored value (or a value it is computed from) was produced inside a loop that does not
    enclose the store: a tile carried from one iteration to the next, or out of its loop.  A loop body is traced
    once, so such a value stands for a single iteration; only the matmul patterns, which read a sum over the
    loop out of it, may accept one."""
    seen = set()
    stack = [value]
    while stack:
        v = stack.pop()
        if id(v) in seen:
            continue
        seen.add(id(v))
        if isinstance(v, Tile):
            v = v.node
        if isinstance(v, Node):
            if id(v) in stop:            # (a matmul accumulator: the matmul matchers read it as a sum over its loop)
                continue
            if len(v.loops) > len(loops) or any(a is not b for a, b in zip(v.loops, loops)):
                return True
            stack.extend(v.args)
            stack.extend(a for a in v.attrs.values() if isinstance(a, (Tile, PlainValue)))
        elif isinstance(v, PlainValue) and v.op not in ("const", "sym"):
            stack.extend(v.args)
    return False


def _loads_of(value: Any) -> List[Node]:
    """The load nodes the value is computed from."""
    found: List[Node] = []
    seen = set()
    stack = [value]
    while stack:
        v = stack.pop()
        if id(v) in seen:
            continue
        seen.add(id(v))
        if isinstance(v, Tile):
            v = v.node
        if isinstance(v, Node):
            if v.kind in ("load", "load_scalar"):
                found.append(v)
            stack.extend(v.args)
            stack.extend(a for a in v.attrs.values() if isinstance(a, (Tile, PlainValue)))
        elif isinstance(v, PlainValue) and v.op not in ("const", "sym"):
            stack.extend(v.args)
    return found


def _split_concat_store(eff: Effect) -> List[Effect]:
    """A store of ``concat(a, b, ...)`` (python/asc/language/tile/creation_ops.py:56-72: tiles joined along the
    first dimension) writes each part at its row offset inside the stored window, so it is planned as one store
    per part; nested concats unfold the same way."""
    value, out_t = eff.args
    if not isinstance(value, Tile) or value.node.kind != "concat":
        return [eff]
    parts = []
    row = 0
    offsets = eff.attrs["offsets"]
    for part in value.node.args:
        attrs = dict(eff.attrs)
        attrs["offsets"] = (offsets[0] + row, ) + tuple(offsets[1:])
        kind = "store_scalar" if part.size == 1 else "store"
        piece = Effect(kind, (part, out_t), attrs, eff.loops, eff.guards)
        piece.uid = eff.uid            # the parts take the place of the store in program order
        parts += _split_concat_store(piece)
        row += part.shape[0]
    return parts


def build_plan(trace: KernelTrace) -> Plan:
    """The C-ABI calls that reproduce the traced kernel's effect on global memory."""
    def is_store(e: Effect) -> bool:
        # scalars and one-element tiles go through the scalar form of asc2.store: a store of one element
        return e.kind in ("store", "store_scalar")
    stores = []
    for e in trace.effects:
        if e.kind == "store":
            stores += _split_concat_store(e)
        elif is_store(e) or e.kind == "atomic":
            stores.append(e)
    others = [e for e in trace.effects if not is_store(e) and e.kind not in ("matmul_acc", "atomic")]
    if others:
        raise _unsupported(f"'{others[0].kind}' side effect")
    if not stores:
        raise _unsupported("kernel without a tile store")
    total = Plan("")
    names = []
    written: Dict[int, int] = {}       # runtime-argument index -> uid of the first effect that writes it
    windows: Dict[int, list] = {}      # runtime-argument index -> (offsets, shape, loop nest) of every store to it
    writers: Dict[int, List[Effect]] = {}   # runtime-argument index -> the planned effects that write it, in order
    footprints: Dict[int, Any] = {}    # id(effect) -> its instances and the rectangles they write (computed on demand)
    for eff in stores:
        if eff.kind != "atomic" and _is_identity_store(eff):
            continue        # a tile stored back to where it was loaded from changes nothing
        plan = None
        scalar_value = not isinstance(eff.args[0], Tile)
        # The plan runs effect after effect, each over all blocks and iterations.  A tile that the kernel loaded
        # *before* an earlier effect overwrote its tensor would be read after that write here: refuse.
        for ld in _loads_of(eff.args[0]):
            src = ld.args[0]
            first_write = written.get(src.base.index) if isinstance(src, Tensor) else None
            if first_write is not None and ld.uid < first_write:
                raise _unsupported(f"kernel '{trace.fn_name}' uses a tile it loaded before an earlier store to the same "
                                   "tensor")
            if first_write is not None and (trace.core_num > 1 or eff.loops or ld.loops):
                # data an earlier effect produced: every block and iteration must read exactly the window it wrote
                # itself, otherwise "all of effect A, then all of effect B" differs from the kernel's own order
                for w_offsets, w_shape, w_loops in windows.get(src.base.index, []):
                    same = (ld.kind == "load" and tuple(ld.attrs["shape"]) == tuple(w_shape) and w_loops == ld.loops
                            and _same_offsets(ld.attrs["offsets"], w_offsets))
                    if not same:
                        raise _unsupported(f"kernel '{trace.fn_name}' reads a tensor back at other positions than an "
                                           "earlier store of the same kernel wrote")
        matchers = (_match_atomic, ) if eff.kind == "atomic" else (_match_eltwise_program, _match_row_scalar) if scalar_value \
            else _MATCHERS
        carried = _value_from_deeper_loop(eff.args[0], eff.loops)
        if carried:
            # only the matmul patterns read a loop-carried value as a sum over the loop
            matchers = tuple(m for m in matchers if m in (_match_matmul, _match_attention, _match_matmul_then_program))
        for matcher in matchers:
            plan = matcher(trace, eff)
            if plan is not None:
                break
        if plan is None and carried:
            raise _unsupported(f"tile carried across iterations of a loop (or out of it) in kernel '{trace.fn_name}'; "
                               "only matmul accumulation over a loop is recognised")
        if plan is None:
            value = eff.args[0]
            kind = value.node.kind if isinstance(value, Tile) else type(value).__name__
            raise _unsupported(f"store of a tile produced by '{kind}' in kernel '{trace.fn_name}'")
        for earlier in writers.get(eff.args[1].base.index, []):
            _check_effect_order(trace, earlier, eff, footprints)
        writers.setdefault(eff.args[1].base.index, []).append(eff)
        written.setdefault(eff.args[1].base.index, eff.uid)
        stored = eff.args[0]
        windows.setdefault(eff.args[1].base.index, []).append(
            (eff.attrs["offsets"], stored.shape if isinstance(stored, Tile) else (1, ), eff.loops))
        names.append(plan.pattern)
        total.steps += plan.steps
        total.reads |= plan.reads
        total.writes |= plan.writes
        total.partial_writes |= plan.partial_writes
        for k, v in plan.temps.items():
            if k in total.temps:
                raise _unsupported("several stores that each need temporary buffers")
            total.temps[k] = v
    if not names:
        raise _unsupported("kernel whose only stores write tiles back unchanged")
    total.pattern = "+".join(names)
    if len(names) == 1 and not total.temps:
        total.pipeline = plan.pipeline
    total.reads = {i for i in total.reads if isinstance(i, int)}
    total.writes = {i for i in total.writes if isinstance(i, int)}
    total.partial_writes = {i for i in total.partial_writes if isinstance(i, int)}
    return total
