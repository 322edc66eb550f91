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
def _col_tag(self) -> int:
    return _COLUMN_TAG.get(self.dtype.name, 4)


Column.dtype_name = lambda self: {1: "f64", 2: "i64", 3: "bool", 4: "str"}[_col_tag(self)]
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
Column.is_f64 = lambda self: _col_tag(self) == 1
Column.is_i64 = lambda self: _col_tag(self) == 2
Column.is_bool = lambda self: _col_tag(self) == 3
Column.is_str = lambda self: _col_tag(self) == 4
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


# ---- MultiIndex (multiindex.mojo:98-480): levels + codes view over the stored tuples ----------------------------------------
_MI_SEP = "\x1f"


def _mi_levels(self):
    """Per level, the distinct labels in first-seen order."""
    out = []
    for lv in range(self.nlevels()):
        seen = []
        for t in self.tuples:
            if t[lv] not in seen:
                seen.append(t[lv])
        out.append(seen)
    return out


def _mi_codes(self):
    lev = _mi_levels(self)
    return [[lev[lv].index(t[lv]) for t in self.tuples] for lv in range(self.nlevels())]


def _mi_from_arrays(arrays, names=None) -> MultiIndex:
    """One array per level; arrays of unequal length give an empty index."""
    arrays = [list(a) for a in arrays]
    if arrays and any(len(a) != len(arrays[0]) for a in arrays):
        return MultiIndex([], None)
    m = MultiIndex(arrays, None)
    _mi_set_names(m, list(names or []))
    return m


def _mi_from_product(levels, names=None) -> MultiIndex:
    import itertools
    m = MultiIndex.from_tuples(list(itertools.product(*[list(l) for l in levels])) if levels else [], None)
    m._n = len(levels)
    _mi_set_names(m, list(names or []))
    return m


def _mi_nlevels(self) -> int:
    return len(self.tuples[0]) if self.tuples else getattr(self, "_n", len(self.names))


def _mi_set_names(self, names):
    L = self.nlevels()
    self.names = [names[i] if i < len(names) else f"level_{i}" for i in range(L)]
    return self


def _mi_rename_levels(self, mapper):
    m = dict(mapper)
    self.names = [m.get(n, n) for n in self.names]
    return self


def _mi_reorder(self, order):
    """A permutation of the levels; anything else leaves the index as it is."""
    L = self.nlevels()
    if sorted(order) != list(range(L)):
        return self
    self.tuples = [tuple(t[i] for i in order) for t in self.tuples]
    self.names = [self.names[i] for i in order]
    return self


def _mi_swaplevel(self, a: int, b: int):
    order = list(range(self.nlevels()))
    if 0 <= a < len(order) and 0 <= b < len(order):
        order[a], order[b] = order[b], order[a]
    return _mi_reorder(self, order)


def _mi_sub(self, rows) -> MultiIndex:
    m = MultiIndex.from_tuples([self.tuples[i] for i in rows], list(self.names))
    m._n = self.nlevels()
    return m


def _mi_is_lexsorted(self) -> bool:
    codes = list(zip(*_mi_codes(self))) if self.tuples else []
    return all(codes[i - 1] <= codes[i] for i in range(1, len(codes)))


MultiIndex.from_arrays = staticmethod(_mi_from_arrays)
MultiIndex.from_product = staticmethod(_mi_from_product)
MultiIndex.nlevels = _mi_nlevels
MultiIndex.nrows = lambda self: len(self.tuples)
MultiIndex.levels_copy = _mi_levels
MultiIndex.codes_copy = _mi_codes
MultiIndex.names_copy = lambda self: list(self.names)
MultiIndex.values = lambda self: [_MI_SEP.join(str(v) for v in t) for t in self.tuples]
MultiIndex.to_index_pair = lambda self: (self.values(), ",".join(self.names))
MultiIndex.set_names, MultiIndex.rename_levels = _mi_set_names, _mi_rename_levels
MultiIndex.reorder_levels, MultiIndex.swaplevel = _mi_reorder, _mi_swaplevel
MultiIndex.take_rows = lambda self, positions: _mi_sub(self, [p for p in positions if 0 <= p < len(self.tuples)])
MultiIndex.mask_rows = lambda self, mask: _mi_sub(self, [i for i, k in enumerate(mask) if k and i < len(self.tuples)])
MultiIndex.level_index_of = lambda self, level, label: (_mi_levels(self)[level].index(label)
                                                        if 0 <= level < self.nlevels() and label in _mi_levels(self)[level] else -1)
MultiIndex.code_of = lambda self, level, row: (_mi_codes(self)[level][row]
                                               if 0 <= level < self.nlevels() and 0 <= row < len(self.tuples) else -1)
MultiIndex.label_of = lambda self, level, row: (str(self.tuples[row][level])
                                                if 0 <= level < self.nlevels() and 0 <= row < len(self.tuples) else "")
MultiIndex.is_lexsorted = _mi_is_lexsorted
MultiIndex.is_unique = lambda self: len(set(self.tuples)) == len(self.tuples)


# ---- Agg as the reference's tagged enum (_groupby_core.mojo:33-190) ----------------------------------------------------------
_AGG_NAMES = ["mean", "sum", "min", "max", "count", "std", "var", "median", "first", "last", "any", "all"]
_AGG_ALIASES = {"avg": "mean", "average": "mean", "total": "sum", "minimum": "min", "maximum": "max", "size": "count",
                "len": "count", "stdev": "std", "stddev": "std", "variance": "var", "p50": "median", "head": "first",
                "tail": "last"}
O._AGG.setdefault("var", lambda x: (Series(x).std() ** 2) if len(x) > 1 else F.NaN)
O._AGG.setdefault("any", lambda x: any(bool(v) for v in x))
O._AGG.setdefault("all", lambda x: all(bool(v) for v in x))


def _agg_make(fn: str):
    return staticmethod(lambda col="", out=None: O.Agg(col, fn, out))


def _agg_parse(name: str):
    """By name or alias, case-insensitive; unknown names give ``mean`` like the reference."""
    n = name.lower()
    n = _AGG_ALIASES.get(n, n)
    return O.Agg("", n if n in _AGG_NAMES else "mean")


for _fn in _AGG_NAMES:
    setattr(O.Agg, {"max": "max_", "var": "var_"}.get(_fn, _fn), _agg_make(_fn))
    setattr(O.Agg, "is_" + _fn, (lambda self, _fn=_fn: self.fn == _fn))
O.Agg.tag = property(lambda self: _AGG_NAMES.index(self.fn) if self.fn in _AGG_NAMES else -1)
O.Agg.name = lambda self: self.fn if self.fn in _AGG_NAMES else "unknown"
O.Agg.parse = staticmethod(_agg_parse)


# ---- query records (utils.mojo:320-432) ------------------------------------------------------------------------------------
R.ExprKind.SINGLE = R.ExprKind.PRED
R.ConstVal.of_f64 = staticmethod(lambda x: R.ConstVal(True, float(x), ""))
R.ConstVal.of_i64 = staticmethod(lambda x: R.ConstVal(True, float(int(x)), ""))
R.ConstVal.of_bool = staticmethod(lambda x: R.ConstVal(True, 1.0 if x else 0.0, ""))
R.ConstVal.of_str = staticmethod(lambda s: R.ConstVal(False, 0.0, str(s)))


def _expr_leaf(p):
    return R.Expr(R.ExprKind.PRED, p)


def _expr_pair(kind):
    return staticmethod(lambda a, b: R.Expr(kind, None, _expr_leaf(a), _expr_leaf(b)))


R.Expr.single = staticmethod(_expr_leaf)
R.Expr.both_and, R.Expr.both_or = _expr_pair(R.ExprKind.AND), _expr_pair(R.ExprKind.OR)
# the reference also lists these under Pred's block, so both spellings resolve
for _cls in (R.Expr, R.Pred):
    _cls.single, _cls.expr_single = staticmethod(_expr_leaf), staticmethod(_expr_leaf)
    _cls.both_and, _cls.expr_and = _expr_pair(R.ExprKind.AND), _expr_pair(R.ExprKind.AND)
    _cls.both_or, _cls.expr_or = _expr_pair(R.ExprKind.OR), _expr_pair(R.ExprKind.OR)


# ---- column comparisons that give row masks (selection.mojo:720-736) --------------------------------------------------------
def _cbo_mask(values, pred):
    return R.Mask([(not isna(v)) and bool(pred(v)) for v in values])


R.ColumnBoolOps.ge = staticmethod(lambda values, value: _cbo_mask(values, lambda v: v >= value))
R.ColumnBoolOps.isin = staticmethod(lambda values, items: _cbo_mask(values, lambda v: v in set(items) or str(v) in set(map(str, items))))
R.ColumnBoolOps.between = staticmethod(lambda values, lo, hi: _cbo_mask(values, lambda v: lo <= v <= hi))


def _doc_push_line(self, name: str, dtype: str) -> None:
    self.rows.append((name, dtype))


R.DTypesDoc.push_line = _doc_push_line


# ---- DataFrame (frame.mojo:153-200, 376-430, 526-700, 800-960, 1161-1360, 1418-1630) ----------------------------------------
def _df_find_col(self, name: str) -> int:
    names = self.col_names()
    return names.index(name) if name in names else -1


def _df_require_col_index(self, name: str) -> int:
    idx = _df_find_col(self, name)
    if idx < 0:
        raise KeyError("Column not found: " + name)
    return idx


def _df_get_column(self, name: str) -> Column:
    """The column, or an empty string-typed one with that name when the frame has none."""
    idx = _df_find_col(self, name)
    return self.columns[idx] if idx >= 0 else Column(name, [], F.string)


def _df_get_column_by_index(self, idx: int) -> Column:
    return self.columns[idx] if 0 <= idx < len(self.columns) else Column()


def _df_put_column(self, col: Column) -> None:
    """Insert, or replace the column of the same name."""
    idx = _df_find_col(self, col.name)
    if idx >= 0:
        self.columns[idx] = col
    else:
        self.columns.append(col)
        if len(self.index) != self.nrows():
            self.index = Index(range(self.nrows()))


def _df_set_column(self, name, rhs=None) -> None:
    """``set_column(column)`` inserts or replaces; ``set_column(name, frame)`` takes the frame's column of that name
    (or its only column) when the row counts agree, else does nothing."""
    if isinstance(name, Column) and rhs is None:
        return _df_put_column(self, name)
    if isinstance(rhs, DataFrame):
        if rhs.nrows() != self.nrows():
            return
        j = _df_find_col(rhs, name)
        if j < 0:
            if rhs.ncols() != 1:
                return
            j = 0
        src = rhs.columns[j]
        return _df_put_column(self, Column(name, list(src.values), src.dtype))
    _df_put_column(self, Column(name, list(rhs)))


def _df_set_columns(self, names, rhs: DataFrame) -> None:
    """Several columns at once: by position from ``rhs``, or its single column broadcast to every name."""
    if rhs.nrows() != self.nrows() or not (rhs.ncols() == 1 or rhs.ncols() == len(names)):
        return
    for k, n in enumerate(names):
        src = rhs.columns[0 if rhs.ncols() == 1 else k]
        _df_put_column(self, Column(n, list(src.values), src.dtype))


def _df_set_rows(self, mask, rhs) -> None:
    """Overwrite the rows where ``mask`` is true with a scalar or with the same rows of ``rhs``."""
    if len(mask) != self.nrows():
        return
    if isinstance(rhs, DataFrame):
        if rhs.nrows() != self.nrows() or not (rhs.ncols() in (1, self.ncols())):
            return
        for c, col in enumerate(self.columns):
            src = rhs.columns[0 if rhs.ncols() == 1 else c].values
            col.values = [src[r] if mask[r] else v for r, v in enumerate(col.values)]
    else:
        for col in self.columns:
            col.values = [rhs if mask[r] else v for r, v in enumerate(col.values)]


def _df_cell_frame(self, r: int, j: int, cname: str) -> DataFrame:
    ok = 0 <= r < self.nrows() and 0 <= j < self.ncols()
    out = DataFrame({cname: [self.columns[j].values[r] if ok else ""]}, [self.index[r] if 0 <= r < self.nrows() else ""])
    return out


def _df_at(self, label_row, col: str) -> DataFrame:
    """1x1 frame for (row label, column name); an empty-string cell when either is unknown."""
    labs = [str(l) for l in self.index.labels]
    r = labs.index(str(label_row)) if str(label_row) in labs else -1
    return _df_cell_frame(self, r, _df_find_col(self, col), col)


def _df_iat(self, row: int, col: int) -> DataFrame:
    return _df_cell_frame(self, row, col, self.col_names()[col] if 0 <= col < self.ncols() else "")


def _df_get(self) -> str:
    """Text of the single cell of a 1-column frame (as ``at`` / ``iat`` return); "" otherwise."""
    if self.ncols() == 1 and self.nrows() > 0:
        return _fmt_cell(self.columns[0].values[0])
    return ""


def _df_set(self, v) -> bool:
    if self.ncols() != 1:
        return False
    self.columns[0].values = [v.v if isinstance(v, Value) else v]
    self.index = Index(self.index.labels[:1] or [0])
    return True


def _df_set_at(self, label_row, col: str, v) -> bool:
    labs = [str(l) for l in self.index.labels]
    j = _df_find_col(self, col)
    if str(label_row) not in labs or j < 0:
        return False
    self.columns[j].values[labs.index(str(label_row))] = v.v if isinstance(v, Value) else v
    return True


def _df_set_iat(self, row: int, col: int, v) -> bool:
    if not (0 <= row < self.nrows() and 0 <= col < self.ncols()):
        return False
    self.columns[col].values[row] = v.v if isinstance(v, Value) else v
    return True


def _df_with_rows(self, n: int) -> DataFrame:
    return self._select_rows_by_positions(list(range(max(0, min(n, self.nrows())))))


def _df_drop_duplicates(self, subset=None, keep: str = "first") -> DataFrame:
    names = list(subset) if subset else self.col_names()
    keys = [tuple(self.col(n).values[i] for n in names) for i in range(self.nrows())]
    if keep == "last":
        last = {k: i for i, k in enumerate(keys)}
        mask = [last[k] == i for i, k in enumerate(keys)]
    elif keep in ("none", "False", False):
        cnt = {}
        for k in keys:
            cnt[k] = cnt.get(k, 0) + 1
        mask = [cnt[k] == 1 for k in keys]
    else:
        seen, mask = set(), []
        for k in keys:
            mask.append(k not in seen)
            seen.add(k)
    return self._select_rows_by_mask(mask)


def _df_assign(self, mapping) -> DataFrame:
    """New or replaced columns from ``name -> values`` or ``name -> function(frame)``, applied in name order."""
    out = self.copy()
    for name in sorted(mapping):
        v = mapping[name]
        v = v(out) if callable(v) else v
        if isinstance(v, (str, bytes, int, float, bool)) or v is None:
            v = [v] * out.nrows()      # a scalar (strings included) fills the whole column
        _df_put_column(out, Column(name, list(v)))
    return out


def _df_from_series(self, src: Series) -> None:
    """Make this frame the one-column frame of ``src`` (its name, values and index)."""
    self.columns = [Column(src.name or "0", list(src.values), src.dtype)]
    self.index = Index(list(src.index.labels))


def _df_to_csv(self, path: str, header: bool = True, delimiter: str = ",", quotechar: str = '"', index: bool = True) -> bool:
    try:
        from .extras import to_csv_string
        with open(path, "w") as f:
            f.write(to_csv_string(self, delimiter, header))
        return True
    except OSError:
        return False


def _df_to_string(self) -> str:
    s = f"DataFrame({self.nrows()}x{self.ncols()})\n"
    iname = getattr(self, "index_name", "") or self.index.name
    s += (iname + " | " if iname else "") + " | ".join(self.col_names()) + "\n"
    for i in range(self.nrows()):
        cells = [_fmt_cell(c.values[i]) if not isna(c.values[i]) else "None" for c in self.columns]
        s += ((str(self.index[i]) + " | ") if iname else "") + " | ".join(cells) + "\n"
    return s


def _sel_rows(df, rows):
    if rows is None or isinstance(rows, R.RowAll) or rows is R.RowAll:
        return None
    if isinstance(rows, R.PosSlice):
        return list(range(*slice(rows.start, rows.stop, getattr(rows, "step", 1) or 1).indices(df.nrows())))
    if isinstance(rows, R.Mask):
        return [i for i, k in enumerate(rows.bits) if k]
    if isinstance(rows, slice):
        return list(range(*rows.indices(df.nrows())))
    if isinstance(rows, int):
        return [rows]
    return list(rows)


def _df_iloc(self, rows=None, cols=None):
    """``iloc(rows, cols)`` by position: markers (``RowAll`` / ``ColAll``), slices, lists or single ints; a single int
    column gives the ``Column``."""
    d = self
    if not (cols is None or isinstance(cols, R.ColAll) or cols is R.ColAll):
        if isinstance(cols, int):
            col = d.columns[cols] if 0 <= cols < d.ncols() else Column()
            r = _sel_rows(d, rows)
            return col if r is None else _col_take(col, r)
        pos = list(range(*cols.indices(d.ncols()))) if isinstance(cols, slice) else list(cols)
        d = d._select_cols_by_positions([c for c in pos if 0 <= c < d.ncols()])
    r = _sel_rows(d, rows)
    return d.copy() if r is None else d._select_rows_by_positions([i for i in r if 0 <= i < d.nrows()])


def _df_loc(self, rows=None, cols=None):
    """``loc(rows, cols)`` by label: row labels (list, ``LabelSlice`` or marker) and column names (or positions)."""
    d = self
    if not (cols is None or isinstance(cols, R.ColAll) or cols is R.ColAll):
        if isinstance(cols, str):
            cols = [cols]
        cols = list(cols)
        d = d._select_cols_by_positions(cols) if cols and isinstance(cols[0], int) else \
            d._select_cols_by_names([c for c in cols if d.has_col(c)])
    if rows is None or isinstance(rows, R.RowAll) or rows is R.RowAll:
        return d.copy()
    if isinstance(rows, R.LabelSlice):
        return d._select_rows_by_positions(R.resolve_label_slice(d.index.labels, rows))
    if isinstance(rows, R.Mask):
        return d._select_rows_by_mask(list(rows.bits))
    labs = [str(l) for l in d.index.labels]
    rows = [rows] if isinstance(rows, (str, int)) else list(rows)
    return d._select_rows_by_positions([labs.index(str(l)) for l in rows if str(l) in labs])


DataFrame.clone = DataFrame.copy
DataFrame.width = lambda self: self.ncols()
DataFrame.height = lambda self: self.nrows()
DataFrame.shape_str = lambda self: f"({self.nrows()}, {self.ncols()})"
DataFrame.find_col = DataFrame.col_index = _df_find_col
DataFrame.require_col_index = _df_require_col_index
DataFrame.get_column = DataFrame.get_column_by_name = _df_get_column
DataFrame.get_column_by_index = _df_get_column_by_index
DataFrame.col_values = lambda self, name: [_fmt_cell(v) for v in _df_get_column(self, name).values]
DataFrame.add_column = _df_put_column
DataFrame.set_column, DataFrame.set_columns, DataFrame.set_rows = _df_set_column, _df_set_columns, _df_set_rows
DataFrame.at, DataFrame.iat, DataFrame.get, DataFrame.set = _df_at, _df_iat, _df_get, _df_set
DataFrame.set_at, DataFrame.set_iat = _df_set_at, _df_set_iat
DataFrame.with_rows = _df_with_rows
DataFrame.drop_duplicates = _df_drop_duplicates
DataFrame.assign = _df_assign
DataFrame.pipe = lambda self, f: f(self.copy())
DataFrame.from_series = _df_from_series
DataFrame.melt = lambda self, id_vars, var_name="variable", value_name="value": O.melt(self, id_vars, var_name, value_name)
DataFrame.merge = lambda self, right, on, how="inner": O.merge(self, right, on, how)
DataFrame.pivot_table = lambda self, index, columns, values, aggfunc="mean", fill_value=None: \
    O.pivot_table(self, index, columns, values, aggfunc, fill_value)
DataFrame.resample = lambda self, freq: R.Resampler(self, freq)
DataFrame.to_csv, DataFrame.to_string = _df_to_csv, _df_to_string
DataFrame.iloc, DataFrame.loc = _df_iloc, _df_loc


# ---- dtype constructor functions (api.mojo:184-200): ``int64(nullable=False)`` gives a ``DType`` ---------------------------
class _DTypeCtor(DType):
    """The package-level ``bool_ / int32 / int64 / float32 / float64 / string``: equal to the plain dtype of that name
    and, called like the reference's constructor functions, a ``DType`` with the requested nullability."""

    def __call__(self, nullable: bool = False) -> DType:
        return _dtype_with_nullable(DType(self.name), nullable)


DTYPE_CONSTRUCTORS = {n: _DTypeCtor(n) for n in _TAGS}
