"""Scalar converters and typed tensor casts under the reference's names
(legacy/src/momijo/tensor/cast.mojo:99-1260). The reference spells out one function per (source, target)
pair because its tensors are not generic at run time; here the pairs are generated from one rule:

* to an integer type: truncate toward zero, then wrap to the type's width (two's complement);
  NaN and infinities give 0;
* to float32 / float16: round to that precision (the result is a Python float holding the rounded value);
* to bool: anything non-zero (NaN included) is True;
* the ``Optional`` helpers (``some_*``, ``opt_*``) keep ``None`` as ``None``.

Names: ``to_<dst>_from_<src>``, ``to_f64_<src>``, ``f32_to_<dst>`` / ``f64_to_<dst>``, ``id_<type>``,
``to_float32_of`` / ``to_float64_of``, and ``astype_<dst>_from_<src>`` for whole tensors."""
from __future__ import annotations

import math
import struct
import sys

import torch

from .cast import astype

_INT_BITS = {"i8": (8, True), "i16": (16, True), "i32": (32, True), "i64": (64, True), "int": (64, True),
             "u8": (8, False), "u16": (16, False), "u32": (32, False), "u64": (64, False), "uint": (64, False)}
_LONG = {"int8": "i8", "int16": "i16", "int32": "i32", "int64": "i64", "int": "int", "uint8": "u8", "uint16": "u16",
         "uint32": "u32", "uint64": "u64", "uint": "uint", "float16": "f16", "float32": "f32", "float64": "f64",
         "bool": "bool"}
_SRC = ["f16", "f32", "f64", "i8", "i16", "i32", "i64", "int", "u8", "u16", "u32", "u64", "uint", "bool",
        "float32", "float64"]


def _to_int(x, bits: int, signed: bool) -> int:
    f = float(x)
    if f != f or math.isinf(f):
        return 0
    v = int(f) & ((1 << bits) - 1)
    return v - (1 << bits) if signed and v >= 1 << (bits - 1) else v


def _to_f32(x) -> float:
    f = float(x)
    if f != f or math.isinf(f):
        return f
    try:
        return struct.unpack("<f", struct.pack("<f", f))[0]
    except OverflowError:
        return math.copysign(math.inf, f)


def _to_f16(x) -> float:
    f = float(x)
    if f != f or math.isinf(f):
        return f
    try:
        return struct.unpack("<e", struct.pack("<e", f))[0]
    except OverflowError:
        return math.copysign(math.inf, f)


def _converter(dst: str):
    dst = _LONG.get(dst, dst)
    if dst in _INT_BITS:
        bits, signed = _INT_BITS[dst]
        return lambda x: _to_int(x, bits, signed)
    if dst == "f64":
        return lambda x: float(x)
    if dst == "f32":
        return _to_f32
    if dst == "f16":
        return _to_f16
    if dst == "bool":
        return lambda x: bool(x != 0) if not isinstance(x, bool) else x
    raise KeyError(dst)


_mod = sys.modules[__name__]
_DSTS = ["f16", "f32", "f64", "i8", "i16", "i32", "i64", "int", "u8", "u16", "u32", "u64", "uint", "bool"]
for _d in _DSTS:
    for _s in _SRC:
        setattr(_mod, f"to_{_d}_from_{_s}", _converter(_d))
for _s in _SRC:
    setattr(_mod, f"to_f64_{_s}", _converter("f64"))
    setattr(_mod, f"to_float32_from_{_s}", _converter("f32"))
    setattr(_mod, f"to_float64_from_{_s}", _converter("f64"))
for _src in ("f32", "f64"):
    for _long, _short in _LONG.items():
        setattr(_mod, f"{_src}_to_{_long}", _converter(_short))
    setattr(_mod, f"{_src}_to", _converter(_src))
for _t in ["f16", "f32", "f64", "i8", "i16", "i32", "i64", "int", "u8", "u16", "u32", "u64", "uint", "bool"]:
    setattr(_mod, f"id_{_t}", lambda x: x)


def to_float32_of(v) -> float:
    return _to_f32(1.0 if v is True else 0.0 if v is False else v)


def to_float64_of(v) -> float:
    return float(v)


to_float32_of_T, to_float64_of_T = to_float32_of, to_float64_of


def val_f64(v, i: int = None) -> float:
    """``float(v)``, or element ``i`` of a list as a float (legacy/src/momijo/tensor/cast.mojo:5341-5346)."""
    return float(v) if i is None else float(v[i])


def from_float64_to(x: float, f):
    """Apply the converter ``f`` to a float64 value."""
    return f(x)


class TypeTag:
    """Carries the float64 -> T converter of a target type."""

    def __init__(self, from_f64):
        self.from_f64 = from_f64


def some_f32(v): return None if v is None else _to_f32(v)         # noqa: E704
def some_f64(v): return None if v is None else float(v)           # noqa: E704
def some_i(v): return None if v is None else int(v)               # noqa: E704
def opt_f32_to_f64(v): return None if v is None else float(v)     # noqa: E704
def opt_i_to_f32(v): return None if v is None else _to_f32(v)     # noqa: E704
def opt_i_to_f64(v): return None if v is None else float(v)       # noqa: E704


def astype_f32_from_f64(x): return astype(x, torch.float32)       # noqa: E704
def astype_f32_from_int(x): return astype(x, torch.float32)       # noqa: E704
def astype_f64_from_f32(x): return astype(x, torch.float64)       # noqa: E704
def astype_f64_from_int(x): return astype(x, torch.float64)       # noqa: E704


def tensor_core_print_nd(x, name: str = "") -> str:
    """Nested-list text of a tensor with a ``name: shape`` header line; also printed."""
    from .tensor import _raw
    t = _raw(x)
    text = f"{name + ': ' if name else ''}shape={list(t.shape)} dtype={str(t.dtype).replace('torch.', '')}\n{t.tolist()}"
    print(text)
    return text


tensor_core_print = tensor_core_print_nd
