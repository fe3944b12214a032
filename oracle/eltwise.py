"""CPU restatement of the elementwise postfix programs (test infrastructure, never on a product path).

The CUDA platform compiles an asc2 elementwise expression (python/asc/language/tile/binary_ops.py,
unary_ops.py, indexing_ops.py:19-27 in the reference) into a postfix program for
``asc_cuda_eltwise_program``.  This module evaluates such a program with torch CPU tensors, one op at
a time, so that tests can check both halves separately: the compiler (program vs. the torch
expression the reference's tests use as golden) and the kernel (device result vs. this evaluator).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

LOAD, CONST, WHERE, ROUND_F16, ROUND_BF16 = 0, 1, 32, 33, 34
_F_BINARY = {2: torch.add, 3: torch.sub, 4: torch.mul, 5: torch.div, 6: torch.maximum, 7: torch.minimum}
_F_UNARY = {
    8: torch.neg, 9: torch.abs, 10: torch.relu, 11: torch.exp, 12: torch.exp2, 13: torch.log, 14: torch.log2,
    15: torch.sqrt, 16: torch.rsqrt, 17: torch.sin, 18: torch.cos, 19: torch.tan, 20: torch.sinh, 21: torch.cosh,
    22: torch.tanh, 23: torch.erf, 24: torch.floor, 25: torch.ceil,
}
_COMPARE = {0: torch.eq, 1: torch.ne, 2: torch.gt, 3: torch.ge, 4: torch.lt, 5: torch.le}
_I_BINARY = {35: torch.add, 36: torch.sub, 37: torch.mul, 38: torch.maximum, 39: torch.minimum,
             40: torch.bitwise_left_shift, 41: torch.bitwise_right_shift}
_I_UNARY = {48: torch.neg, 49: torch.abs, 50: torch.relu}
_F_SWAPPED = {54: torch.sub, 55: torch.div}
_I_SWAPPED = {56: torch.sub, 57: torch.bitwise_left_shift, 58: torch.bitwise_right_shift}
_ROW = {59: lambda t: t.sum(-1, keepdim=True), 60: lambda t: t.amax(-1, keepdim=True),
        61: lambda t: t.amin(-1, keepdim=True), 62: lambda t: t.prod(-1, keepdim=True)}
IMM = 0x100
INDEX = 65                 # the element's row-major index inside the window, as int32
TYPES = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16, 3: torch.int32, 4: torch.int16}


def run_program(ops: Sequence[int], args: Sequence[int], inputs: List[torch.Tensor], out_type: int) -> torch.Tensor:
    """Evaluates the program over whole tensors.  Stack entries are fp32 or int32 tensors; a CONST's
    kind (float bits or integer) is resolved when the first op consumes it, as on the device where
    the word is untyped."""
    shape = inputs[0].shape
    stack: list = []
    tmp: dict = {}

    def as_float(v):
        return v if isinstance(v, torch.Tensor) else torch.tensor([v], dtype=torch.int32).view(torch.float32).expand(shape)

    def as_int(v):
        return v if isinstance(v, torch.Tensor) else torch.tensor([v], dtype=torch.int32).expand(shape)

    for op, arg in zip(ops, args):
        if op & IMM:                          # left operand is the word in arg: put it under the top
            stack.insert(len(stack) - 1, int(arg))
            op &= 0xff
        if op == LOAD:
            t = inputs[arg]
            stack.append(t.to(torch.int32) if not t.dtype.is_floating_point else t.to(torch.float32))
        elif op == CONST:
            stack.append(int(arg))            # untyped 32-bit word
        elif op == INDEX:
            stack.append(torch.arange(inputs[0].numel(), dtype=torch.int32).reshape(shape))
        elif op in _F_BINARY:
            b, a = as_float(stack.pop()), as_float(stack.pop())
            stack.append(_F_BINARY[op](a, b))
        elif 26 <= op <= 31:
            b, a = as_float(stack.pop()), as_float(stack.pop())
            stack.append(_COMPARE[op - 26](a, b).to(torch.float32))
        elif op in _I_BINARY:
            b, a = as_int(stack.pop()), as_int(stack.pop())
            stack.append(_I_BINARY[op](a, b))
        elif 42 <= op <= 47:
            b, a = as_int(stack.pop()), as_int(stack.pop())
            stack.append(_COMPARE[op - 42](a, b).to(torch.float32))
        elif op in _F_SWAPPED:
            b, a = as_float(stack.pop()), as_float(stack.pop())
            stack.append(_F_SWAPPED[op](b, a))
        elif op in _I_SWAPPED:
            b, a = as_int(stack.pop()), as_int(stack.pop())
            stack.append(_I_SWAPPED[op](b, a))
        elif op == WHERE:
            b, a, c = stack.pop(), stack.pop(), as_float(stack.pop())
            int_kind = any(isinstance(v, torch.Tensor) and v.dtype == torch.int32 for v in (a, b)) or out_type in (3, 4)
            conv = as_int if int_kind else as_float
            stack.append(torch.where(c != 0, conv(a), conv(b)))
        elif op in _F_UNARY:
            stack.append(_F_UNARY[op](as_float(stack.pop())))
        elif op == ROUND_F16:
            stack.append(as_float(stack.pop()).to(torch.float16).to(torch.float32))
        elif op == ROUND_BF16:
            stack.append(as_float(stack.pop()).to(torch.bfloat16).to(torch.float32))
        elif op in _I_UNARY:
            stack.append(_I_UNARY[op](as_int(stack.pop())))
        elif op == 51:
            stack.append(as_int(stack.pop()).to(torch.float32))
        elif op == 52:
            stack.append(torch.trunc(as_float(stack.pop())).to(torch.int32))
        elif op == 53:
            stack.append(as_int(stack.pop()).to(torch.int16).to(torch.int32))
        elif op == 63:                        # TEE: copy the top into temporary slot arg
            tmp[int(arg)] = stack[-1]
        elif op == 64:                        # TMP: push temporary slot arg
            stack.append(tmp[int(arg)])
        elif op in _ROW:
            # row programs (asc_cuda_row_program): the reduction over the last dimension replaces every element
            t = as_float(stack.pop()).expand(shape)
            stack.append(_ROW[op](t.double()).to(torch.float32).expand(shape))
        else:
            raise ValueError(f"unknown opcode {op}")
    assert len(stack) == 1, "malformed program"
    top = stack[0]
    dtype = TYPES[out_type]
    top = (as_float if dtype.is_floating_point else as_int)(top)
    return top.expand(shape).to(dtype)
