"""Element types of the asc/asc2 surface (reference: python/asc/language/core/dtype.py:19-153).

Only what asc2 kernels touch is provided: a ``DataType`` value type with name / width / kind
queries and the module-level instances ``asc.float16`` ... ``asc.int64``.
"""
from __future__ import annotations

from typing import Any, Dict

_BITS: Dict[str, int] = {
    "bool": 1, "int8": 8, "int16": 16, "int32": 32, "int64": 64,
    "uint8": 8, "uint16": 16, "uint32": 32, "uint64": 64,
    "float16": 16, "bfloat16": 16, "float32": 32, "float64": 64,
}
_ALIASES = {"half": "float16", "float": "float32", "double": "float64", "int": "int32", "bool_": "bool"}


class DataType:
    """A named scalar type; equal when names are equal."""

    def __init__(self, name: Any):
        if isinstance(name, DataType):
            name = name.name
        name = str(name)
        if name.startswith("torch."):
            name = name[6:]
        name = _ALIASES.get(name, name)
        if name not in _BITS:
            raise ValueError(f"Unknown data type: {name}")
        self.name = name

    @property
    def bitwidth(self) -> int:
        return _BITS[self.name]

    def sizeof(self) -> int:
        if self.bitwidth < 8:
            raise ValueError(f"sizeof is not defined for {self.name}")
        return self.bitwidth // 8

    def is_float(self) -> bool:
        return self.name in ("float16", "bfloat16", "float32", "float64")

    def is_signed(self) -> bool:
        return self.name in ("int8", "int16", "int32", "int64")

    def is_unsigned(self) -> bool:
        return self.name.startswith("uint")

    def is_int(self) -> bool:
        return self.is_signed() or self.is_unsigned()

    def is_bool(self) -> bool:
        return self.name == "bool"

    def to_numpy(self):
        import numpy as np
        if self.name == "bfloat16":
            raise TypeError("NumPy has no bfloat16")
        return np.dtype("bool" if self.name == "bool" else self.name)

    def to_torch(self):
        import torch
        return getattr(torch, self.name)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, DataType) and other.name == self.name

    def __hash__(self) -> int:
        return hash(("asc.DataType", self.name))

    def __str__(self) -> str:
        return self.name

    def __repr__(self) -> str:
        return f"asc.{self.name}"


class KnownTypes:
    bool_ = DataType("bool")
    int8 = DataType("int8")
    int16 = DataType("int16")
    int32 = DataType("int32")
    int64 = DataType("int64")
    uint8 = DataType("uint8")
    uint16 = DataType("uint16")
    uint32 = DataType("uint32")
    uint64 = DataType("uint64")
    float16 = DataType("float16")
    half = float16
    bfloat16 = DataType("bfloat16")
    float32 = DataType("float32")
    float_ = float32
    float64 = DataType("float64")
    int_ = int32


bool_ = KnownTypes.bool_
int8 = KnownTypes.int8
int16 = KnownTypes.int16
int32 = KnownTypes.int32
int64 = KnownTypes.int64
uint8 = KnownTypes.uint8
uint16 = KnownTypes.uint16
uint32 = KnownTypes.uint32
uint64 = KnownTypes.uint64
float16 = KnownTypes.float16
half = KnownTypes.float16
bfloat16 = KnownTypes.bfloat16
float32 = KnownTypes.float32
float64 = KnownTypes.float64

__all__ = ["DataType", "KnownTypes", "bool_", "int8", "int16", "int32", "int64", "uint8", "uint16", "uint32",
           "uint64", "float16", "half", "bfloat16", "float32", "float64"]
