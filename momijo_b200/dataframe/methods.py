"""The reference's method spellings on the dataframe classes (legacy/src/momijo/dataframe/api.mojo:65-142, 780-916,
bitmap.mojo:32-190, column.mojo:105-700, series_*.mojo, multiindex.mojo, frame.mojo, _groupby_core.mojo). The classes
keep Python lists with ``None`` for missing cells; these methods give them the call forms of the reference
(``col.dtype()`` tag, ``series.values()``, ``bitmap.count_true()`` ...) on top of that storage."""
from __future__ import annotations

from typing import List, Sequence

from . import frame as F
from . import ops as O
from . import relational as R
from .frame import Bitmap, Column, DataFrame, DType, Index, MultiIndex, Series, Value, isna

# ---- DType: tag + nullable (api.mojo:65-142) -----------------------------------------------------------------------------
_TAGS = {"bool": 1, "int32": 2, "int64": 3, "float32": 4, "float64": 5, "string": 6}
_TAG_NAMES = {v: k for k, v in _TAGS.items()}
_COLUMN_TAG = {"float32": 1, "float64": 1, "int32": 2, "int64": 2, "bool": 3, "string": 4}   # ColumnTag F64/I64/BOOL/STR


def _dtype_tag(self) -> int:
    return _TAGS.get(self.name, 0)


def _dtype_with_nullable(self, make_nullable: bool) -> DType:
    d = DType(self.name)
    d.nullable = bool(make_nullable)
    return d


def _dtype_ctor(name: str):
    def make(nullable: bool = False) -> DType:
        return _dtype_with_nullable(DType(name), nullable)
    return staticmethod(make)


DType.tag = property(_dtype_tag)
DType.nullable = False
DType.with_nullable = _dtype_with_nullable
DType.is_nullable = lambda self: bool(self.nullable)
DType.__call__ = lambda self: _COLUMN_TAG.get(self.name, 4)     # ``column.dtype()`` is the column's storage tag
for _n, _t in _TAGS.items():
    setattr(DType, "is_" + _n, (lambda self, _n=_n: self.name == _n))
    setattr(DType, "tag_" + {"float32": "f32", "float64": "f64"}.get(_n, _n), staticmethod(lambda _t=_t: _t))
    setattr(DType, _n.upper(), _dtype_ctor(_n))


# ---- Bitmap (bitmap.mojo:32-190) ------------------------------------------------------------------------------------------
def _bm_set(self, i: int, v: bool = True) -> bool:
    """False (and no change) for an index outside the map."""
    if not 0 <= i < len(self.bits):
        return False
    self.bits[i] = bool(v)
    return True


def _bm_resize(self, n: int, fill: bool = False) -> None:
    n = max(n, 0)
    self.bits = self.bits[:n] + [bool(fill)] * (n - len(self.bits))


def _bm_zip(a: Bitmap, b: Bitmap, fn) -> Bitmap:
    out = Bitmap(min(len(a.bits), len(b.bits)), False)
    out.bits = [fn(x, y) for x, y in zip(a.bits, b.bits)]
    return out


def _bm_from_mask(mask) -> Bitmap:
    out = Bitmap(0)
    out.bits = [bool(v) for v in mask]
    return out


Bitmap.__len__ = lambda self: len(self.bits)
Bitmap.len = lambda self: len(self.bits)
Bitmap.get = lambda self, i: bool(self.bits[i]) if 0 <= i < len(self.bits) else False
Bitmap.set = _bm_set
Bitmap.is_set = Bitmap.get
Bitmap.count_true = lambda self: sum(1 for b in self.bits if b)
Bitmap.count_false = lambda self: sum(1 for b in self.bits if not b)
Bitmap.any_true = lambda self: any(self.bits)
Bitmap.none_true = lambda self: not any(self.bits)
Bitmap.to_mask = lambda self: [bool(b) for b in self.bits]
Bitmap.resize = _bm_resize
Bitmap.invert = lambda self: setattr(self, "bits", [not b for b in self.bits])
Bitmap.bit_and = lambda self, o: _bm_zip(self, o, lambda x, y: bool(x and y))
Bitmap.bit_or = lambda self, o: _bm_zip(self, o, lambda x, y: bool(x or y))
Bitmap.all_true = staticmethod(lambda n: Bitmap(n, True))
Bitmap.all_false = staticmethod(lambda n: Bitmap(n, False))
Bitmap.from_mask = staticmethod(_bm_from_mask)
Bitmap.__str__ = lambda self: "Bitmap(" + "".join("1" if b else "0" for b in self.bits) + ")"


# ---- Value (column.mojo:653-705) -------------------------------------------------------------------------------------------
def _fmt_cell(v) -> str:
    if isna(v):
        return ""
    if isinstance(v, bool):
        return "True" if v else "False"
    return str(v)


Value.as_string = lambda self: _fmt_cell(self.v)
Value.int32 = staticmethod(lambda x: Value(int(x)))
Value.int64 = staticmethod(lambda x: Value(int(x)))
Value.float64 = staticmethod(lambda x: Value(float(x)))
Value.bool = staticmethod(lambda x: Value(bool(x)))


# ---- values() / index() call forms on Series -------------------------------------------------------------------------------
class _Values(list):
    """The series' cells: a list that also answers the reference's ``series.values()`` call with a copy."""

    def __call__(self):
        return list(self)


def _get_values(self):
    return self._values


def _set_values(self, vals):
    self._values = vals if isinstance(vals, _Values) else _Values(vals)


Series.values = property(_get_values, _set_values)
Index.__call__ = lambda self: list(self.labels)            # ``series.index()`` gives the labels


# ---- typed series (series_bool / i64 / f64 / str .mojo) ---------------------------------------------------------------------
def _ts_like(self, vals):
    out = type(self)(vals, self.name)
    return out


def _ts_set(self, i: int, value, is_valid: bool = True) -> None:
    if 0 <= i < len(self.values):
        self.values[i] = self._conv(value) if is_valid and not isna(value) else None


def _ts_append(self, value, is_valid: bool = True) -> None:
    self.values.append(self._conv(value) if is_valid and not isna(value) else None)
    self.index.labels.append(len(self.values) - 1)


def _ts_take(self, idxs):
    """Rows by position; a position outside the series gives the type's zero (0, 0.0, False, "")."""
    zero = self._conv(0) if self._conv is not str else ""
    return _ts_like(self, [self.values[j] if 0 <= j < len(self.values) else zero for j in idxs])


def _ts_gather(self, mask):
    m = mask.to_mask() if isinstance(mask, Bitmap) else list(mask)
    return _ts_like(self, [v for v, keep in zip(self.values, m) if keep])


def _ts_validity(self) -> Bitmap:
    return Bitmap.from_mask([not isna(v) for v in self.values])


def _ts_resize(self, n: int) -> None:
    n = max(n, 0)
    cur = len(self.values)
    self.values = list(self.values[:n]) + [None] * (n - cur)
    self.index.labels = list(range(n))


def _ts_clear(self) -> None:
    self.values = []
    self.index.labels = []


def _ts_extend(self, more) -> None:
    for v in more:
        _ts_append(self, v)


_TS = R._TypedSeries
_TS.clone = _TS.copy = lambda self: _ts_like(self, list(self.values))
_TS.set, _TS.append, _TS.take, _TS.gather, _TS.validity = _ts_set, _ts_append, _ts_take, _ts_gather, _ts_validity
_TS.set_name = lambda self, name: setattr(self, "name", name)
_TS.get_name = lambda self: self.name
_TS.head = lambda self, k: _ts_like(self, list(self.values[:max(k, 0)]))
_TS.count_valid = lambda self: sum(1 for v in self.values if not isna(v))
_TS.null_count = lambda self: sum(1 for v in self.values if isna(v))
_TS.is_empty = lambda self: len(self.values) == 0
_TS.set_null = lambda self, i: _ts_set(self, i, None, False)
_TS.resize, _TS.clear, _TS.extend = _ts_resize, _ts_clear, _ts_extend
_TS.to_string = lambda self: f"{type(self).__name__}(name={self.name}, values={list(self.values)})"
Series.to_string = lambda self: f"Series(name={self.name}, values={list(self.values)})"


def _sb_binary(a, b, fn):
    """Element-wise on the common length; a missing operand gives a missing result."""
    n = min(len(a.values), len(b.values))
    return R.SeriesBool([None if isna(a.values[i]) or isna(b.values[i]) else fn(a.values[i], b.values[i])
                         for i in range(n)], a.name)


R.SeriesBool.sum_true = lambda self: sum(1 for v in self.values if v is True)
R.SeriesBool.logical_not = lambda self: R.SeriesBool([None if isna(v) else (not v) for v in self.values], self.name)
R.SeriesBool.logical_and = lambda self, o: _sb_binary(self, o, lambda x, y: x and y)
R.SeriesBool.logical_or = lambda self, o: _sb_binary(self, o, lambda x, y: x or y)
R.SeriesBool.logical_xor = lambda self, o: _sb_binary(self, o, lambda x, y: x != y)
R.SeriesI64.mean_as_f64 = lambda self: Series.mean(self)


# ---- Column (column.mojo:105-580) ------------------------------------------------------------------------------------------
def _col_from_series(self, src) -> None:
    self.values = list(src.values)
    self.dtype = F._infer_dtype(self.values) if not isinstance(src, R._TypedSeries) else \
        {R.SeriesF64: F.float64, R.SeriesI64: F.int64, R.SeriesBool: F.bool_, R.SeriesStr: F.string}[type(src)]
    if getattr(src, "name", ""):
        self.name = src.name


def _col_take(self, idxs) -> Column:
    return Column(self.name, [self.values[j] if 0 <= j < len(self.values) else None for j in idxs], self.dtype)


def _col_gather(self, mask) -> Column:
    m = mask.to_mask() if isinstance(mask, Bitmap) else list(mask)
    return Column(self.name, [v for v, keep in zip(self.values, m) if keep], self.dtype)


def _col_to_string(self, show: int = 10) -> str:
    cells = [_fmt_cell(v) if not isna(v) else "None" for v in self.values[:max(show, 0)]]
    more = ", ..." if len(self.values) > show else ""
    return f"Column(name={self.name}, dtype={self.dtype_name()}, n={len(self.values)}, values=[{', '.join(cells)}{more}])"


Column.clone = Column.copy
Column.dtype_name = lambda self: {1: "f64", 2: "i64", 3: "bool", 4: "str"}[self.dtype()]
Column.len = lambda self: len(self.values)
Column.is_valid = lambda self, i: 0 <= i < len(self.values) and not isna(self.values[i])
Column.null_count = lambda self: sum(1 for v in self.values if isna(v))
Column.value_str = lambda self, i: _fmt_cell(self.values[i]) if 0 <= i < len(self.values) else ""
Column.get_str = Column.get_string = Column.value_str
Column.get_bool = lambda self, i: bool(self.values[i]) if 0 <= i < len(self.values) and not isna(self.values[i]) else False
Column.from_str = Column.from_i64 = Column.from_f64 = Column.from_bool = _col_from_series
Column.set_string_series = Column.set_bool_series = Column.set_f64_series = Column.set_i64_series = _col_from_series
Column.rename = lambda self, new_name: setattr(self, "name", new_name)
Column.get_name = lambda self: self.name
Column.is_f64 = lambda self: self.dtype() == 1
Column.is_i64 = lambda self: self.dtype() == 2
Column.is_bool = lambda self: self.dtype() == 3
Column.is_str = lambda self: self.dtype() == 4
Column.take, Column.gather = _col_take, _col_gather
Column.null_mask = lambda self: R.SeriesBool([isna(v) for v in self.values], self.name)
Column.has_none = lambda self: any(isna(v) for v in self.values)
Column.is_none = lambda self: len(self.values) == 0
Column.all_none = lambda self: len(self.values) > 0 and all(isna(v) for v in self.values)
Column.value = lambda self: self.copy()
Column.to_string = _col_to_string
Column.__str__ = lambda self: _col_to_string(self)


# ---- ColPair / IndexPair (api.mojo:780-916) -----------------------------------------------------------------------------------
def _cp_make(kind: int):
    def make(name: str, values) -> "R.ColPair":
        return R.ColPair(name, list(values), kind)
    return staticmethod(make)


def _cp_get(self, i: int) -> str:
    """Clamped read as text; "" for an empty pair."""
    if not self.values:
        return ""
    return str(self.values[min(max(i, 0), len(self.values) - 1)])


R.ColPair.of_str, R.ColPair.of_i64, R.ColPair.of_f64 = _cp_make(R.ColKind.STR), _cp_make(R.ColKind.I64), _cp_make(R.ColKind.F64)
R.ColPair.of = _cp_make(R.ColKind.STR)
R.ColPair.empty = staticmethod(lambda name: R.ColPair(name, []))
R.ColPair.single = staticmethod(lambda name, value: R.ColPair(name, [value]))
R.ColPair.len = lambda self: len(self.values)
R.ColPair.is_empty = lambda self: len(self.values) == 0
R.ColPair.get = _cp_get
R.ColPair.push = lambda self, value: self.values.append(value)
R.ColPair.extend = lambda self, more: self.values.extend(more)
R.ColPair.clear = lambda self: self.values.clear()
R.IndexPair.copy = lambda self: R.IndexPair(self.pos, self.label)
