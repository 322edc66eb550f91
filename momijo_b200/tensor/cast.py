"""Dtype conversions (legacy/src/momijo/tensor/cast.mojo:656-5310): the 13 x 8 conversion matrix
collapses to ``astype``; float -> int truncates toward zero, anything -> bool is ``!= 0``."""
from __future__ import annotations

import torch

from .tensor import _wrap, _raw


def astype(x, dtype):
    if isinstance(dtype, str):
        from .dtype import from_name

        dtype = from_name(dtype).torch()
    elif hasattr(dtype, "torch") and not isinstance(dtype, torch.dtype):
        dtype = dtype.torch()
    r = _raw(x)
    if dtype == torch.bool:
        return _wrap(r != 0)
    if r.dtype.is_floating_point and not dtype.is_floating_point:
        r = torch.nan_to_num(torch.trunc(r), nan=0.0)
    return _wrap(r.to(dtype))


def to_float64(x): return astype(x, torch.float64)
def to_float32(x): return astype(x, torch.float32)
def to_float16(x): return astype(x, torch.float16)
def to_bfloat16(x): return astype(x, torch.bfloat16)
def to_int(x): return astype(x, torch.int64)
def to_int64(x): return astype(x, torch.int64)
def to_int32(x): return astype(x, torch.int32)
def to_int16(x): return astype(x, torch.int16)
def to_int8(x): return astype(x, torch.int8)
def to_uint8(x): return astype(x, torch.uint8)
def to_bool(x): return astype(x, torch.bool)


def to_string(x) -> str:
    from .printing import tensor_to_string

    return tensor_to_string(x)
