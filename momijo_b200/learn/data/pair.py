"""``Pair``: one image sample, a [C, H, W] tensor ``x`` with its class index ``y``
(legacy/src/momijo/learn/data/pair.mojo:14-58). ``first`` / ``second`` alias the two fields so the pair also
unpacks as a tuple."""
from __future__ import annotations

from typing import Any, List


class Pair:
    def __init__(self, x: Any = None, y: Any = None, first: Any = None, second: Any = None):
        self.x = x if x is not None else first
        self.y = y if y is not None else second

    first = property(lambda self: self.x)
    second = property(lambda self: self.y)

    @staticmethod
    def empty() -> "Pair":
        import torch

        return Pair(torch.zeros(1, 1, 1), 0)

    @staticmethod
    def from_xy(x, y) -> "Pair":
        return Pair(x, y)

    def shape(self) -> List[int]:
        return list(self.x.shape) if hasattr(self.x, "shape") else []

    def _dim(self, k: int) -> int:
        shp = self.shape()
        return shp[k] if len(shp) > k else 0

    def channels(self) -> int:
        return self._dim(0)

    def height(self) -> int:
        return self._dim(1)

    def width(self) -> int:
        return self._dim(2)

    def is_valid(self) -> bool:
        shp = self.shape()
        return len(shp) == 3 and all(d > 0 for d in shp)

    def __iter__(self):
        yield self.x
        yield self.y

    def __eq__(self, o):
        return isinstance(o, Pair) and self.y == o.y and (self.x is o.x or bool((self.x == o.x) if not hasattr(self.x, "shape") else (self.shape() == o.shape() and bool((self.x == o.x).all()))))

    def __str__(self):
        return f"Pair(shape={self.shape()}, y={self.y})"

    __repr__ = __str__
