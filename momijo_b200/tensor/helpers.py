"""Stride / contiguity / selector helpers (legacy/src/momijo/tensor/helpers.mojo)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .tensor import _raw, _wrap


def compute_row_major_strides(shape) -> List[int]:
    s, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        s[i] = acc
        acc *= max(int(shape[i]), 1)
    return s


mk_strides = compute_row_major_strides


def is_contiguous(shape, strides) -> bool:
    return list(strides) == compute_row_major_strides(shape)


def numel(shape) -> int:
    n = 1
    for v in shape:
        n *= int(v)
    return n


@dataclass
class SliceSpec:
    start: Optional[int] = None
    stop: Optional[int] = None
    step: Optional[int] = None

    def to_slice(self):
        return slice(self.start, self.stop, self.step)


@dataclass
class IndexSel:
    """One selector: an integer index, a slice, or a list of indices (fancy)."""
    index: Optional[int] = None
    slice: Optional[SliceSpec] = None
    fancy: Optional[List[int]] = None

    def to_key(self):
        if self.index is not None:
            return self.index
        if self.fancy is not None:
            return list(self.fancy)
        return (self.slice or SliceSpec()).to_slice()


def normalize_slice_1d(n: int, start, stop, step):
    """Python slice normalisation including negative steps."""
    return slice(start, stop, step).indices(n)


def select(x, sels: List[IndexSel]):
    return _wrap(_raw(x)[tuple(s.to_key() for s in sels)])


def write_plane(x, axis: int, index: int, plane):
    """x.select(axis, index) = plane (in place); returns x."""
    _raw(x).select(axis, index).copy_(_raw(plane))
    return x


class XorShift64:
    def __init__(self, seed: int = 88172645463325252):
        self.s = (seed or 88172645463325252) & ((1 << 64) - 1)

    def next_u64(self) -> int:
        x = self.s
        x ^= (x << 13) & ((1 << 64) - 1)
        x ^= x >> 7
        x ^= (x << 17) & ((1 << 64) - 1)
        self.s = x
        return x

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)


def sort_values(x, descending=False):
    return _wrap(torch.sort(_raw(x).reshape(-1), descending=descending, stable=True).values)


def argsort_values(x, descending=False):
    return _wrap(torch.argsort(_raw(x).reshape(-1), descending=descending, stable=True))


def unique_values(x):
    return _wrap(torch.unique(_raw(x)))
