"""``asc2``: the tile-based, NumPy-like front end (reference: python/asc2/__init__.py:9-95).
Same public names; ``causal_mask`` and the ``trans_b`` / int8 forms of ``matmul`` are extensions of
the CUDA platform."""
from asc.language.tile.tensor import tensor
from asc.language.tile.tile import TileLocation
from asc.language.tile.range import range
from asc.language.tile.atomic_ops import atomic_add, atomic_max, atomic_min
from asc.language.tile.binary_ops import (add, div, equal, greater, greater_equal, left_shift, less, less_equal,
                                          matmul, matmul_acc, maximum, minimum, mul, not_equal, right_shift, sub)
from asc.language.tile.creation_ops import concat, full, full_like, zeros, zeros_acc, zeros_like
from asc.language.tile.memory_ops import copy, load, store
from asc.language.tile.prog_model_ops import block_idx, block_num, num_tiles
from asc.language.tile.shape_ops import broadcast_to, expand_dims, ravel, reshape, squeeze
from asc.language.tile.unary_ops import (abs, ceil, cos, cosh, erf, exp, exp2, floor, log, log2, negative, relu,
                                         rms_norm, rsqrt, sin, sinh, softmax, sqrt, tan, tanh)
from asc.language.tile.indexing_ops import causal_mask, mask, where
from asc.language.tile.reduction_ops import reduce_max, reduce_min, reduce_prod, reduce_sum

from .jit import jit

__all__ = [
    "tensor",
    "TileLocation",
    "range",
    "atomic_add",
    "atomic_max",
    "atomic_min",
    "add",
    "div",
    "equal",
    "greater",
    "greater_equal",
    "left_shift",
    "less",
    "less_equal",
    "matmul",
    "matmul_acc",
    "maximum",
    "minimum",
    "mul",
    "not_equal",
    "right_shift",
    "sub",
    "concat",
    "full",
    "full_like",
    "zeros",
    "zeros_acc",
    "zeros_like",
    "copy",
    "load",
    "store",
    "block_idx",
    "block_num",
    "num_tiles",
    "broadcast_to",
    "expand_dims",
    "ravel",
    "reshape",
    "squeeze",
    "abs",
    "ceil",
    "cos",
    "cosh",
    "erf",
    "exp",
    "exp2",
    "floor",
    "log",
    "log2",
    "negative",
    "relu",
    "rms_norm",
    "rsqrt",
    "sin",
    "sinh",
    "softmax",
    "sqrt",
    "tan",
    "tanh",
    "mask",
    "where",
    "reduce_max",
    "reduce_min",
    "reduce_sum",
    "reduce_prod",
    "causal_mask",
    "jit",
]
