"""Datasets (legacy/src/momijo/learn/data/dataset.mojo:48-597): list wrappers with
map/filter/concat, tuple / iterable / index-view / zip / enumerate datasets and the LCG
Fisher-Yates shuffle ``state * 1664525 + 1013904223`` used by the loaders."""
from __future__ import annotations

from typing import Callable, Iterable, List


def lcg_shuffle(n: int, seed: int) -> List[int]:
    """Fisher-Yates with the reference LCG (dataset.mojo:570-597)."""
    idx = list(range(n))
    state = seed & 0xFFFFFFFF
    for i in range(n - 1, 0, -1):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        j = state % (i + 1)
        idx[i], idx[j] = idx[j], idx[i]
    return idx


class Dataset:
    def __init__(self, items=None):
        self.items = list(items) if items is not None else []

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]

    def get(self, i):
        return self.items[i]

    def append(self, x):
        self.items.append(x)
        return self

    def map(self, fn: Callable):
        return Dataset([fn(x) for x in self.items])

    def filter(self, pred: Callable):
        return Dataset([x for x in self.items if pred(x)])

    def concat(self, other: "Dataset"):
        return Dataset(self.items + list(other.items))

    def take(self, n: int):
        return Dataset(self.items[:n])

    def skip(self, n: int):
        return Dataset(self.items[n:])

    def shuffle(self, seed: int = 42):
        order = lcg_shuffle(len(self.items), seed)
        return Dataset([self.items[i] for i in order])

    def to_list(self):
        return list(self.items)

    def __iter__(self):
        return iter(self.items)


class TupleDataset(Dataset):
    """Pairs ``(x, y)`` built from two parallel sequences."""

    def __init__(self, xs, ys):
        if len(xs) != len(ys):
            raise ValueError("length mismatch")
        super().__init__(list(zip(xs, ys)))


class TensorDataset(Dataset):
    """Rows of one or more tensors that share dim 0; ``get_batch(step)`` serves the Trainer."""

    def __init__(self, *tensors):
        n = tensors[0].shape[0]
        if any(t.shape[0] != n for t in tensors):
            raise ValueError("tensors must share dim 0")
        self.tensors = tensors
        self.items = range(n)

    def __getitem__(self, i):
        return tuple(t[i] for t in self.tensors)

    get = __getitem__


class IterableDataset:
    def __init__(self, source: Iterable | Callable[[], Iterable]):
        self.source = source

    def __iter__(self):
        return iter(self.source() if callable(self.source) else self.source)

    def map(self, fn):
        src = self
        return IterableDataset(lambda: (fn(x) for x in src))

    def filter(self, pred):
        src = self
        return IterableDataset(lambda: (x for x in src if pred(x)))

    def take(self, n):
        src = self

        def gen():
            for i, x in enumerate(src):
                if i >= n:
                    break
                yield x
        return IterableDataset(gen)


class IndexSliceDataset(Dataset):
    def __init__(self, base, start: int, end: int):
        self.base, self.start, self.end = base, start, min(end, len(base))
        self.items = range(self.start, self.end)

    def __getitem__(self, i):
        return self.base[self.start + i]

    get = __getitem__


class IndexListDataset(Dataset):
    def __init__(self, base, indices):
        self.base, self.indices = base, list(indices)
        self.items = self.indices

    def __getitem__(self, i):
        return self.base[self.indices[i]]

    get = __getitem__


class ZipDataset(Dataset):
    def __init__(self, a, b):
        self.a, self.b = a, b
        self.items = range(min(len(a), len(b)))

    def __getitem__(self, i):
        return (self.a[i], self.b[i])

    get = __getitem__


class EnumerateDataset(Dataset):
    def __init__(self, base, start: int = 0):
        self.base, self.start0 = base, start
        self.items = range(len(base))

    def __getitem__(self, i):
        return (self.start0 + i, self.base[i])

    get = __getitem__
