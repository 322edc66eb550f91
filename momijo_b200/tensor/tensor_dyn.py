"""Type-erased tensors (legacy/src/momijo/tensor/tensor_dyn.mojo:33-808): ``AnyTensor`` carries a
dtype tag next to the data, ``TensorView`` is a (shape, strides, offset) window on shared data."""
from __future__ import annotations

import torch

from .dtype import DType
from .tensor import _raw, _wrap


class AnyBuffer:
    def __init__(self, data: torch.Tensor):
        self.data = _raw(data).reshape(-1)
        self.dtype = DType.of(self.data)

    def __len__(self):
        return self.data.numel()


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
