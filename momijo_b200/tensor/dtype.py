"""Dtype table: the design that the reference keeps commented out
(legacy/src/momijo/tensor/dtype.mojo:15-308): 13 codes bool..float64, ``DType{tag,itemsize}``,
the promotion lattice bool<u8<i8<i16<u16<i32<u32<i64<u64<f16~bf16<f32<f64, ``can_cast``,
``from_name/to_code/from_code``."""
from __future__ import annotations

from dataclasses import dataclass

import torch


class DTypeTag:
    BOOL, UINT8, INT8, INT16, UINT16, INT32, UINT32, INT64, UINT64, FLOAT16, BFLOAT16, FLOAT32, FLOAT64 = range(13)


_NAMES = ["bool", "uint8", "int8", "int16", "uint16", "int32", "uint32", "int64", "uint64", "float16",
          "bfloat16", "float32", "float64"]
_SIZES = [1, 1, 1, 2, 2, 4, 4, 8, 8, 2, 2, 4, 8]
_TORCH = [torch.bool, torch.uint8, torch.int8, torch.int16, torch.uint16, torch.int32, torch.uint32,
          torch.int64, torch.uint64, torch.float16, torch.bfloat16, torch.float32, torch.float64]
_RANK = [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 9, 10, 11]


@dataclass(frozen=True)
class DType:
    tag: int
    itemsize: int

    @property
    def name(self):
        return _NAMES[self.tag]

    def torch(self):
        return _TORCH[self.tag]

    def is_float(self):
        return self.tag >= DTypeTag.FLOAT16

    def is_int(self):
        return DTypeTag.UINT8 <= self.tag <= DTypeTag.UINT64

    def is_bool(self):
        return self.tag == DTypeTag.BOOL

    def __str__(self):
        return self.name

    @staticmethod
    def of(t) -> "DType":
        dt = t.dtype if hasattr(t, "dtype") else t
        return from_code(_TORCH.index(dt))


def itemsize_for_code(code: int) -> int:
    return _SIZES[code] if 0 <= code < 13 else 0


def from_code(code: int) -> DType:
    return DType(code, itemsize_for_code(code))


def to_code(dt: DType) -> int:
    return dt.tag


def from_name(name: str) -> DType:
    alias = {"int": "int64", "float": "float64", "f32": "float32", "f64": "float64", "i32": "int32",
             "i64": "int64", "u8": "uint8", "bf16": "bfloat16", "f16": "float16", "half": "float16"}
    n = alias.get(name.lower(), name.lower())
    if n not in _NAMES:
        raise ValueError(f"unknown dtype name {name!r}")
    return from_code(_NAMES.index(n))


def promote_dtype(a: DType, b: DType) -> DType:
    if a.tag == b.tag:
        return a
    ra, rb = _RANK[a.tag], _RANK[b.tag]
    if ra == rb:  # float16 vs bfloat16: widen to float32
        return from_code(DTypeTag.FLOAT32)
    hi = a if ra > rb else b
    lo = b if ra > rb else a
    # unsigned 64 with a signed integer has no common integer type: go to float64
    if hi.tag == DTypeTag.UINT64 and lo.tag in (DTypeTag.INT8, DTypeTag.INT16, DTypeTag.INT32, DTypeTag.INT64):
        return from_code(DTypeTag.FLOAT64)
    return hi


def can_cast(src: DType, dst: DType, mode: str = "safe") -> bool:
    """``mode``: "safe" (no information loss by rank), "same_kind" (stay in int/float family or
    widen to float), "unsafe" (anything)."""
    if mode == "unsafe" or src.tag == dst.tag:
        return True
    if mode == "same_kind":
        if src.is_float():
            return dst.is_float()
        return dst.is_int() or dst.is_float() or (src.is_bool() and dst.is_bool())
    if src.is_float() and not dst.is_float():
        return False
    return _RANK[dst.tag] >= _RANK[src.tag] and promote_dtype(src, dst).tag == dst.tag
