"""Datasets (legacy/src/momijo/learn/data/dataset.mojo:48-597): list wrappers with
map/filter/concat, tuple / iterable / index-view / zip / enumerate datasets and the LCG
Fisher-Yates shuffle ``state * 1664525 + 1013904223`` used by the loaders."""
from __future__ import annotations

from typing import Callable, Iterable, List


class LCG32:
    """state <- state * 1664525 + 1013904223 (mod 2^32) (legacy/src/momijo/learn/data/dataset.mojo:570-585)."""

    def __init__(self, seed: int):
        self.state = int(seed) & 0xFFFFFFFF

    def next_u32(self) -> int:
        self.state = (self.state * 1664525 + 1013904223) & 0xFFFFFFFF
        return self.state

    def randint(self, lo: int, hi: int) -> int:
        """Integer in [lo, hi) from the low 31 bits of the next state."""
        span = hi - lo
        if span <= 0:
            return lo
        return lo + (self.next_u32() & 0x7FFFFFFF) % span


def shuffle_inplace(idxs: List[int], seed: int) -> List[int]:
    """Fisher-Yates from the back with ``LCG32(seed)`` (legacy/src/momijo/learn/data/dataset.mojo:588-597)."""
    rng = LCG32(seed)
    for i in range(len(idxs) - 1, 0, -1):
        j = rng.randint(0, i + 1)
        idxs[i], idxs[j] = idxs[j], idxs[i]
    return idxs


def lcg_shuffle(n: int, seed: int) -> List[int]:
    """Shuffled ``range(n)``: ``shuffle_inplace(make_arange(n), seed)``."""
    return shuffle_inplace(list(range(n)), seed)


def make_arange(n: int) -> List[int]:
    return list(range(max(0, n)))


def clamp_index(i: int, n: int) -> int:
    """i clamped into [0, n - 1]; 0 for an empty range."""
    if n <= 0:
        return 0
    return min(max(i, 0), n - 1)


def make_random_index_partition(n: int, train_ratio: float, seed: int):
    """(train indices, validation indices): a seeded shuffle of range(n) cut at int(n * train_ratio)
    (legacy/src/momijo/learn/data/dataset.mojo:599-617)."""
    idxs = lcg_shuffle(n, seed)
    k = min(max(int(float(n) * train_ratio), 0), n)
    return idxs[:k], idxs[k:]


class IndexIter:
    """Cursor over ``range(n)`` (legacy/src/momijo/learn/data/dataset.mojo:307-323)."""

    def __init__(self, n: int):
        self.i, self.n = 0, n

    def reset(self):
        self.i = 0

    def done(self) -> bool:
        return self.i >= self.n


class IndexAdapter:
    """Uniform ``len`` / ``[]`` view of any indexable source, optionally through caller-supplied accessors
    (legacy/src/momijo/learn/data/dataset.mojo:355-388)."""

    def __init__(self, base, len_fn=None, get_fn=None):
        self.base = base
        self._len = len_fn or (lambda b: len(b))
        self._get = get_fn or (lambda b, i: b[i])

    def __len__(self):
        return self._len(self.base)

    def __getitem__(self, idx):
        return self._get(self.base, idx)

    @staticmethod
    def from_dataset(base):
        return IndexAdapter(base)

    @staticmethod
    def from_image_folder(base):
        return IndexAdapter(base)


class Dataset:
    def __init__(self, items=None):
        self.items = list(items) if items is not None else []

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]

    _MISSING = object()

    def get(self, i, default=_MISSING):
        """``get(i)`` indexes; ``get(i, default)`` gives the default outside the range
        (legacy/src/momijo/learn/data/dataset.mojo:94-100)."""
        if default is not Dataset._MISSING and not 0 <= i < len(self.items):
            return default
        return self.items[i]

    def append(self, x):
        self.items.append(x)
        return self

    # ---- list surface of the reference (dataset.mojo:58-175) -------------------------------------------------
    @staticmethod
    def from_list(items) -> "Dataset":
        return Dataset(items)

    def with_items(self, items):
        self.items = list(items)
        return self

    def is_empty(self) -> bool:
        return len(self.items) == 0

    def front(self):
        return self.items[0] if len(self.items) else None

    def back(self):
        return self.items[-1] if len(self.items) else None

    def set(self, idx: int, value) -> None:
        if 0 <= idx < len(self.items):
            self.items[idx] = value

    def extend(self, values) -> None:
        self.items.extend(values)

    def insert(self, idx: int, value) -> None:
        self.items.insert(min(max(idx, 0), len(self.items)), value)

    def pop(self):
        return self.items.pop() if len(self.items) else None

    def clear(self) -> None:
        self.items = []

    def slice(self, start: int, stop: int) -> "Dataset":
        s = max(start, 0)
        e = min(max(stop, s), len(self.items))
        return Dataset(self.items[s:e])

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

    def __init__(self, xs=(), ys=()):
        if len(xs) != len(ys):
            raise ValueError("length mismatch")
        super().__init__(list(zip(xs, ys)))

    # The factory forms truncate to the shorter list instead of raising (dataset.mojo:227-253).
    @staticmethod
    def from_lists(x, y) -> "TupleDataset":
        m = min(len(x), len(y))
        return TupleDataset(list(x)[:m], list(y)[:m])

    def with_lists(self, x, y):
        m = min(len(x), len(y))
        self.items = list(zip(list(x)[:m], list(y)[:m]))
        return self

    def get(self, idx, default_a=Dataset._MISSING, default_b=None):
        if default_a is not Dataset._MISSING and not 0 <= idx < len(self.items):
            return (default_a, default_b)
        return self.items[idx]

    def append(self, a, b=Dataset._MISSING):
        self.items.append(a if b is Dataset._MISSING else (a, b))
        return self

    def to_lists(self):
        return [a for a, _ in self.items], [b for _, b in self.items]

    def to_dataset(self) -> Dataset:
        return Dataset(self.items)


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

    # cursor protocol of the reference (legacy/src/momijo/learn/data/dataset.mojo:334-352)
    def with_dataset(self, data):
        self.source = data
        return self

    def __len__(self):
        return len(self.source)

    def _make_index_iter(self):
        return IndexIter(len(self))

    def next_item(self, it):
        """Item under the cursor (and advance), or None at the end."""
        if it.done():
            return None
        idx = it.i
        it.i += 1
        return self.source[idx]

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


# ---- factories of the reference (legacy/src/momijo/learn/data/dataset.mojo:517-548) ------------------------
def make_index_slice(base, start: int, length: int, mk_empty=None):
    """View of ``length`` items of ``base`` from ``start``. ``mk_empty`` (the reference's filler for
    out-of-range reads) is accepted and unused: out-of-range reads raise IndexError here."""
    return IndexSliceDataset(IndexAdapter(base), start, start + length)


def make_index_list(base, indices, mk_empty=None):
    return IndexListDataset(IndexAdapter(base), indices)


def make_zip(left, right):
    return ZipDataset(IndexAdapter(left), IndexAdapter(right))


def make_enumerate(base):
    return EnumerateDataset(IndexAdapter(base))
