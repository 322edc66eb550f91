"""pandas-like ``DataFrame`` / ``Series`` / ``Column`` without pandas
(legacy/src/momijo/dataframe/frame.mojo:62, column.mojo:51-653, series.mojo, selection.mojo).

Columns are Python lists; missing values are ``None`` (the reference keeps a validity bitmap next
to tagged cells). Numeric columns can be exported to tensors with ``to_tensor``."""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence


class DType:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return self.name

    def __eq__(self, o):
        return isinstance(o, DType) and o.name == self.name

    def __hash__(self):
        return hash(self.name)


int32, int64, bool_, float32, float64, string = (DType(n) for n in
                                                ("int32", "int64", "bool", "float32", "float64", "string"))
NaN = float("nan")
NoneStr = None


def isna(v) -> bool:
    return v is None or (isinstance(v, float) and v != v)


def _infer_dtype(vals) -> DType:
    seen = {type(v) for v in vals if not isna(v)}
    if not seen:
        return float64
    if seen <= {bool}:
        return bool_
    if seen <= {int, bool}:
        return int64
    if seen <= {int, float, bool}:
        return float64
    return string


class Value:
    """Tagged cell (column.mojo:653)."""

    def __init__(self, v=None):
        self.v = v

    def is_null(self):
        return isna(self.v)

    def as_f64(self):
        return float(self.v) if not self.is_null() else NaN

    def as_int(self):
        return int(self.v) if not self.is_null() else 0

    def as_str(self):
        return "" if self.is_null() else str(self.v)

    def __repr__(self):
        return f"Value({self.v!r})"


class Bitmap:
    def __init__(self, n=0, fill=True):
        self.bits = [bool(fill)] * max(n, 0)

    def set(self, i, v=True):
        self.bits[i] = v

    def get(self, i):
        return self.bits[i]

    def count(self):
        return sum(self.bits)


class Column:
    def __init__(self, name: str = "", values: Optional[Iterable] = None, dtype: Optional[DType] = None):
        self.name = name
        self.values = list(values) if values is not None else []
        self.dtype = dtype or _infer_dtype(self.values)

    def __len__(self):
        return len(self.values)

    def __getitem__(self, i):
        return self.values[i]

    def __iter__(self):
        return iter(self.values)

    def copy(self):
        return Column(self.name, list(self.values), self.dtype)

    def validity(self) -> Bitmap:
        b = Bitmap(len(self.values))
        for i, v in enumerate(self.values):
            b.set(i, not isna(v))
        return b

    def get(self, i) -> Value:
        return Value(self.values[i])

    def to_list(self):
        return list(self.values)

    def to_tensor(self, dtype=None):
        import torch

        vals = [NaN if isna(v) else float(v) for v in self.values]
        return torch.tensor(vals, dtype=dtype or torch.float64)

    def __repr__(self):
        return f"Column({self.name!r}, {self.values!r})"


class Index:
    def __init__(self, labels: Iterable = (), name: str = ""):
        self.labels, self.name = list(labels), name

    def __len__(self):
        return len(self.labels)

    def __getitem__(self, i):
        return self.labels[i]

    def get_loc(self, label):
        return self.labels.index(label)

    def to_list(self):
        return list(self.labels)


class MultiIndex:
    def __init__(self, levels: Sequence[Sequence], names: Optional[Sequence[str]] = None):
        self.tuples = list(zip(*levels)) if levels else []
        self.names = list(names) if names else [f"level_{i}" for i in range(len(levels))]

    @staticmethod
    def from_tuples(tuples, names=None):
        m = MultiIndex([], names)
        m.tuples = [tuple(t) for t in tuples]
        if names:
            m.names = list(names)
        return m

    def __len__(self):
        return len(self.tuples)

    def get_level_values(self, i):
        return [t[i] for t in self.tuples]


class Series:
    def __init__(self, values: Iterable = (), index: Optional[Iterable] = None, name: str = "", dtype=None):
        self.values = list(values)
        self.index = Index(index if index is not None else range(len(self.values)))
        self.name = name
        self.dtype = dtype or _infer_dtype(self.values)

    def __len__(self):
        return len(self.values)

    def __getitem__(self, i):
        return self.values[i]

    def __iter__(self):
        return iter(self.values)

    def to_list(self):
        return list(self.values)

    def _num(self):
        return [float(v) for v in self.values if not isna(v)]

    def sum(self):
        return sum(self._num())

    def mean(self):
        x = self._num()
        return sum(x) / len(x) if x else NaN

    def min(self):
        x = self._num()
        return min(x) if x else NaN

    def max(self):
        x = self._num()
        return max(x) if x else NaN

    def std(self, ddof=1):
        x = self._num()
        if len(x) <= ddof:
            return NaN
        m = sum(x) / len(x)
        return math.sqrt(sum((v - m) ** 2 for v in x) / (len(x) - ddof))

    def count(self):
        return len(self._num())

    def map(self, fn):
        return Series([None if isna(v) else fn(v) for v in self.values], self.index.labels, self.name)

    def isna(self):
        return Series([isna(v) for v in self.values], self.index.labels, self.name)

    def fillna(self, v):
        return Series([v if isna(x) else x for x in self.values], self.index.labels, self.name)

    def unique(self):
        out = []
        for v in self.values:
            if v not in out:
                out.append(v)
        return out

    def value_counts(self):
        c = {}
        for v in self.values:
            if not isna(v):
                c[v] = c.get(v, 0) + 1
        return dict(sorted(c.items(), key=lambda kv: -kv[1]))

    def to_tensor(self, dtype=None):
        return Column(self.name, self.values).to_tensor(dtype)

    def __repr__(self):
        return f"Series({self.name!r}, {self.values!r})"


def series_from_list(values, name="", index=None):
    return Series(values, index, name)


def Series_from_strings(values, name=""):
    return Series([str(v) for v in values], None, name, string)


def series_index(s: Series):
    return s.index.to_list()


class DataFrame:
    def __init__(self, data: Optional[Dict[str, Iterable]] = None, index: Optional[Iterable] = None):
        self.columns: List[Column] = []
        if data:
            n = None
            for k, v in data.items():
                col = v if isinstance(v, Column) else Column(k, list(v))
                col.name = k
                if n is None:
                    n = len(col)
                elif len(col) != n:
                    raise ValueError(f"column {k!r} has {len(col)} rows, expected {n}")
                self.columns.append(col)
        self.index = Index(index if index is not None else range(self.nrows()))
        self.index_name = ""

    # ---- shape / access ----
    def nrows(self):
        return len(self.columns[0]) if self.columns else 0

    def ncols(self):
        return len(self.columns)

    def shape(self):
        return (self.nrows(), self.ncols())

    def col_names(self):
        return [c.name for c in self.columns]

    def dtypes(self):
        return {c.name: c.dtype for c in self.columns}

    def has_col(self, name):
        return name in self.col_names()

    def col(self, name) -> Column:
        for c in self.columns:
            if c.name == name:
                return c
        raise KeyError(name)

    def __getitem__(self, key):
        if isinstance(key, str):
            c = self.col(key)
            return Series(c.values, self.index.labels, c.name, c.dtype)
        if isinstance(key, list) and all(isinstance(k, str) for k in key):
            return self._select_cols_by_names(key)
        if isinstance(key, list):
            return self._select_rows_by_mask(key)
        raise KeyError(key)

    def __setitem__(self, name, values):
        vals = list(values.values) if isinstance(values, (Series, Column)) else list(values)
        if self.columns and len(vals) != self.nrows():
            raise ValueError("length mismatch")
        for i, c in enumerate(self.columns):
            if c.name == name:
                self.columns[i] = Column(name, vals)
                return
        self.columns.append(Column(name, vals))
        if len(self.index) != self.nrows():
            self.index = Index(range(self.nrows()))

    def copy(self):
        d = DataFrame()
        d.columns = [c.copy() for c in self.columns]
        d.index = Index(self.index.labels, self.index.name)
        d.index_name = self.index_name
        return d

    def row(self, i) -> dict:
        return {c.name: c.values[i] for c in self.columns}

    def iterrows(self):
        for i in range(self.nrows()):
            yield self.index[i], self.row(i)

    def to_dict(self):
        return {c.name: list(c.values) for c in self.columns}

    def to_records(self):
        return [self.row(i) for i in range(self.nrows())]

    def to_tensor(self, cols=None, dtype=None):
        import torch

        names = cols or [c.name for c in self.columns if c.dtype != string]
        return torch.stack([self.col(n).to_tensor(dtype) for n in names], dim=1)

    # ---- selection helpers used by loc / iloc ----
    def _select_cols_by_names(self, names):
        d = DataFrame({n: list(self.col(n).values) for n in names}, self.index.labels)
        return d

    def _select_cols_by_positions(self, pos):
        return self._select_cols_by_names([self.columns[p].name for p in pos])

    def _select_rows_by_positions(self, rows):
        d = DataFrame({c.name: [c.values[r] for r in rows] for c in self.columns},
                      [self.index[r] for r in rows])
        return d

    def _select_rows_by_mask(self, mask):
        return self._select_rows_by_positions([i for i, m in enumerate(mask) if m])

    def head(self, n=5):
        return self._select_rows_by_positions(list(range(min(n, self.nrows()))))

    def tail(self, n=5):
        N = self.nrows()
        return self._select_rows_by_positions(list(range(max(0, N - n), N)))

    # ---- mutation-free transforms ----
    def sort_values(self, by, ascending=True):
        by = [by] if isinstance(by, str) else list(by)
        asc = [ascending] * len(by) if isinstance(ascending, bool) else list(ascending)
        order = list(range(self.nrows()))
        for name, a in reversed(list(zip(by, asc))):
            vals = self.col(name).values
            order.sort(key=lambda i: (isna(vals[i]), vals[i] if not isna(vals[i]) else 0), reverse=not a)
            if not a:   # keep missing values last
                order = [i for i in order if not isna(vals[i])] + [i for i in order if isna(vals[i])]
        return self._select_rows_by_positions(order)

    def set_index(self, name):
        d = self._select_cols_by_names([n for n in self.col_names() if n != name])
        d.index = Index(self.col(name).values, name)
        d.index_name = name
        return d

    def reset_index(self, name=None):
        d = DataFrame({(name or self.index_name or "index"): list(self.index.labels)})
        for c in self.columns:
            d[c.name] = list(c.values)
        return d

    def rename(self, mapping: Dict[str, str]):
        d = self.copy()
        for c in d.columns:
            c.name = mapping.get(c.name, c.name)
        return d

    def drop(self, names):
        names = [names] if isinstance(names, str) else names
        return self._select_cols_by_names([n for n in self.col_names() if n not in names])

    def describe(self):
        rows = ["count", "mean", "std", "min", "max"]
        out = {"stat": rows}
        for c in self.columns:
            if c.dtype == string:
                continue
            s = Series(c.values)
            out[c.name] = [s.count(), s.mean(), s.std(), s.min(), s.max()]
        return DataFrame(out)

    def __repr__(self):
        names = self.col_names()
        lines = ["\t".join([""] + names)]
        for i in range(min(self.nrows(), 20)):
            lines.append("\t".join([str(self.index[i])] + ["NA" if isna(c.values[i]) else str(c.values[i]) for c in self.columns]))
        if self.nrows() > 20:
            lines.append(f"... ({self.nrows()} rows)")
        return "\n".join(lines)

    __str__ = __repr__
