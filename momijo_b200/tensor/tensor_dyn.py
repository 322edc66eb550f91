"""Type-erased tensors (legacy/src/momijo/tensor/tensor_dyn.mojo:33-808): ``AnyTensor`` carries a
dtype tag next to the data, ``TensorView`` is a (shape, strides, offset) window on shared data."""
from __future__ import annotations

import torch

from .dtype import DType
from .tensor import _raw, _wrap


class AnyBuffer:
    """Flat storage with a dtype tag (tensor_dyn.mojo:56-185)."""

    def __init__(self, data: torch.Tensor = None):
        self.data = _raw(data).reshape(-1) if data is not None else torch.zeros(0, dtype=torch.float64)
        self.dtype = DType.of(self.data)

    @property
    def tag(self) -> int:
        return self.dtype.tag

    def __len__(self):
        return self.data.numel()

    def length(self) -> int:
        return self.data.numel()

    def reserve(self, n: int, tag: int = None) -> None:
        """Only the tag matters here: an empty buffer takes the dtype it will be filled with."""
        if tag is not None and tag != self.tag and self.data.numel() == 0:
            from .dtype import from_code

            self.dtype = from_code(tag)
            self.data = torch.zeros(0, dtype=self.dtype.torch())

    def get_f64(self, i: int) -> float:
        return float(self.data[i])

    def append_cast_from_f64(self, v: float, tag: int = None) -> None:
        """Append one value given as float64, cast by the destination's rule (integers truncate toward zero)."""
        self.reserve(1, tag)
        self.data = torch.cat([self.data, torch.tensor([v], dtype=torch.float64).to(self.data.dtype)])


class AnyTensor:
    def __init__(self, t):
        self.t = _raw(t)

    @property
    def dtype(self) -> DType:
        return DType.of(self.t)

    @property
    def tag(self) -> int:
        return self.dtype.tag

    def shape(self):
        return list(self.t.shape)

    def numel(self):
        return self.t.numel()

    def astype(self, dt):
        from .cast import astype

        return AnyTensor(astype(self.t, dt))

    def to_f64(self):
        return _wrap(self.t.double())

    def to_f32(self):
        return _wrap(self.t.float())

    def to_int(self):
        return _wrap(self.t.long())

    def unwrap(self):
        return _wrap(self.t)

    # ---- the reference's method spellings (tensor_dyn.mojo:187-700) ----------------------------------------
    def strides(self):
        return list(self.t.stride())

    def is_row_major_contiguous(self) -> bool:
        return self.t.is_contiguous()

    def copy(self) -> "AnyTensor":
        return AnyTensor(self.t.clone())

    def astype_inplace(self, dt) -> None:
        self.t = self.astype(dt).t

    def zeros_like_dtype_shape(self, dt, shp) -> None:
        self.t = torch.zeros(list(shp), dtype=dt.torch() if hasattr(dt, "torch") else dt)

    def full_like_dtype_shape(self, dt, shp, value_as_f64: float) -> None:
        self.t = torch.full(list(shp), value_as_f64, dtype=torch.float64).to(dt.torch() if hasattr(dt, "torch") else dt)

    def __repr__(self):
        return f"AnyTensor(dtype={self.dtype}, shape={self.shape()})"


class TensorView:
    def __init__(self, base, shape=None, strides=None, offset: int = 0):
        b = _raw(base)
        self.base = b
        if shape is None:
            self.view = b
        else:
            from .helpers import compute_row_major_strides

            self.view = torch.as_strided(b, list(shape), list(strides or compute_row_major_strides(shape)), offset)

    def shape(self):
        return list(self.view.shape)

    def strides(self):
        return list(self.view.stride())

    def offset(self):
        return self.view.storage_offset()

    def materialize(self):
        return _wrap(self.view.contiguous())

    def tensor(self):
        return _wrap(self.view)

    def to_tensor(self):
        return self.materialize()


def _bind_typed(name: str, torch_dtype) -> None:
    """``from_tensor_<t>`` adopts a tensor as that dtype; ``to_tensor_<t>`` reads the data out as that dtype
    (tensor_dyn.mojo:560-680)."""
    def from_tensor(self, t):
        self.t = _raw(t).to(torch_dtype).clone()

    def to_tensor(self):
        return _wrap(self.t.to(torch_dtype))

    setattr(AnyTensor, "from_tensor_" + name, from_tensor)
    setattr(AnyTensor, "to_tensor_" + name, to_tensor)


for _n, _t in (("f64", torch.float64), ("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16),
               ("i64", torch.int64), ("i32", torch.int32), ("i16", torch.int16), ("i8", torch.int8),
               ("u64", torch.uint64), ("u32", torch.uint32), ("u16", torch.uint16), ("u8", torch.uint8),
               ("bool", torch.bool)):
    _bind_typed(_n, _t)
