"""DataFrame operations: construction helpers, selection (loc/iloc/filter), groupby / Agg / pivot,
joins (merge, merge_asof), missing data, rolling / expanding / EWM, string and datetime helpers,
categorical, CSV / JSON I/O. Public names follow legacy/src/momijo/dataframe/__init__.mojo."""
from __future__ import annotations

import csv
import json
import math
import re
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

from .frame import (Column, DataFrame, DType, Index, Series, Value, NaN, bool_, float32, float64, int32,
                    int64, isna, string, _infer_dtype)


# ---- construction ------------------------------------------------------------------------------------
def make_pairs():
    return []


def pairs_append(pairs, name: str, values):
    return list(pairs) + [(name, list(values))]


def df_from_pairs(pairs) -> DataFrame:
    return DataFrame({n: v for n, v in pairs})


def df_from_columns(names: Sequence[str], cols: Sequence[Sequence]) -> DataFrame:
    return DataFrame({n: list(c) for n, c in zip(names, cols)})


df_make = df_from_columns


def ToDataFrame(data: Dict[str, Iterable], index=None) -> DataFrame:
    """Frame from ``name -> values``; ``index`` gives the row labels (legacy/src/momijo/dataframe/api.mojo:506-660)."""
    return DataFrame(data, index)


def ToDataFrameNullable(data: Dict[str, Iterable], null_token="") -> DataFrame:
    return DataFrame({k: [None if v == null_token else v for v in vs] for k, vs in data.items()})


def df_shape(df):
    return df.shape()


def df_dtypes(df):
    return df.dtypes()


def df_describe(df):
    return df.describe()


def df_rename(df, mapping, axis_name: str = ""):
    """Rename columns from a dict or a list of ``(old, new)`` pairs; a non-empty third argument names the index
    (legacy/src/momijo/dataframe/api.mojo:1213, 2153-2157)."""
    out = df.rename(dict(mapping))
    if axis_name:
        out.index.name = axis_name
    return out


rename = df_rename


def copy(df):
    return df.copy()


def range(start, stop=None, step=1):
    import builtins

    return list(builtins.range(start, stop, step)) if stop is not None else list(builtins.range(start))


def range_f64(start, stop, step=1.0):
    out, v = [], float(start)
    while (step > 0 and v < stop) or (step < 0 and v > stop):
        out.append(v)
        v += step
    return out


def set_col_strings(df, name, values):
    d = df.copy()
    d[name] = [str(v) for v in values]
    return d


def col_from_list_with_tag(name, values, tag):
    cast = {"int": int, "float": float, "str": str, "bool": bool}.get(tag, lambda v: v)
    return Column(name, [None if isna(v) else cast(v) for v in values])


def make_broadcast_col_by_name(df, name, value):
    d = df.copy()
    d[name] = [value] * df.nrows()
    return d


def make_broadcast_col_by_pos(df, pos, value):
    return make_broadcast_col_by_name(df, df.columns[pos].name, value)


def set_value(df, row, col, value):
    d = df.copy()
    d.col(col).values[row] = value
    return d


def set_null(df, row, col):
    return set_value(df, row, col, None)


def assign(df, newcols: Dict[str, Iterable]):
    d = df.copy()
    for k, v in newcols.items():
        if isinstance(v, (str, bytes, int, float, bool)) or v is None:
            v = [v] * df.nrows()       # a scalar (strings included) fills the whole column
        d[k] = list(v)
    return d


assign_flex = assign_numeric = assign_int = assign_bool = assign


def astype(df, col, dtype):
    cast = {"int32": int, "int64": int, "float32": float, "float64": float, "string": str, "bool": bool}[
        dtype.name if isinstance(dtype, DType) else str(dtype)]
    d = df.copy()
    d[col] = [None if isna(v) else cast(v) for v in df.col(col).values]
    return d


def replace_values(df, col, old, new):
    d = df.copy()
    d[col] = [new if v == old else v for v in df.col(col).values]
    return d


def coerce_str_to_f64(df, col):
    def f(v):
        try:
            return float(v)
        except (TypeError, ValueError):
            return None
    d = df.copy()
    d[col] = [f(v) for v in df.col(col).values]
    return d


def take_rows(df, rows):
    return df._select_rows_by_positions(list(rows))


def concat_rows(a, b):
    names = a.col_names() + [n for n in b.col_names() if n not in a.col_names()]
    return DataFrame({n: (list(a.col(n).values) if a.has_col(n) else [None] * a.nrows())
                      + (list(b.col(n).values) if b.has_col(n) else [None] * b.nrows()) for n in names})


def concat_cols(a, b):
    d = a.copy()
    for c in b.columns:
        d[c.name if not d.has_col(c.name) else c.name + "_r"] = list(c.values)
    return d


def melt(df, id_vars, var_name="variable", value_name="value"):
    vals = [n for n in df.col_names() if n not in id_vars]
    out = {n: [] for n in list(id_vars) + [var_name, value_name]}
    for v in vals:
        for i in range(df.nrows()):
            for n in id_vars:
                out[n].append(df.col(n).values[i])
            out[var_name].append(v)
            out[value_name].append(df.col(v).values[i])
    return DataFrame(out)


def cut_numeric(df, col, bins, labels):
    out = []
    for v in df.col(col).values:
        lab = None
        if not isna(v):
            for i in range(len(bins) - 1):
                if bins[i] < v <= bins[i + 1] or (i == 0 and v == bins[0]):
                    lab = labels[i]
                    break
        out.append(lab)
    return out


# ---- selection ------------------------------------------------------------------------------------------
@dataclass
class RowRange:
    start: int = 0
    stop: Optional[int] = None


@dataclass
class ColRange:
    start: int = 0
    stop: Optional[int] = None


def rows_all():
    return None


def cols_all():
    return None


def rows(*idx):
    return list(idx[0]) if len(idx) == 1 and isinstance(idx[0], (list, tuple)) else list(idx)


def pslice(start, stop):
    return RowRange(start, stop)


def select(df, names):
    return df._select_cols_by_names(list(names))


def _rows_of(df, r):
    if r is None:
        return list(range(df.nrows()))
    if isinstance(r, RowRange):
        return list(range(df.nrows()))[r.start:r.stop]
    if isinstance(r, (list, tuple)) and r and isinstance(r[0], bool):
        return [i for i, m in enumerate(r) if m]
    return list(r)


def iloc(df, r=None, c=None):
    d = df._select_rows_by_positions(_rows_of(df, r))
    if c is None:
        return d
    pos = list(range(df.ncols()))[c.start:c.stop] if isinstance(c, ColRange) else list(c)
    return d._select_cols_by_positions(pos)


def loc(df, r=None, c=None):
    if r is not None and not isinstance(r, RowRange) and r and not isinstance(r[0], (bool, int)):
        r = [df.index.get_loc(l) for l in r]     # label based
    d = df._select_rows_by_positions(_rows_of(df, r))
    if c is None:
        return d
    if isinstance(c, str):
        return d.col(c)
    return d._select_cols_by_names(list(c)) if isinstance(c[0], str) else d._select_cols_by_positions(list(c))


def slice_rows(df, start, stop):
    return iloc(df, RowRange(start, stop))


def slice_cols(df, start, stop):
    return iloc(df, None, ColRange(start, stop))


def slice_labels(df, first, last):
    a, b = df.index.get_loc(first), df.index.get_loc(last)
    return iloc(df, RowRange(a, b + 1))


def col_ge(df, col, v):
    return [(not isna(x)) and x >= v for x in df.col(col).values]


def col_isin(df, col, values):
    s = set(values)
    return [x in s for x in df.col(col).values]


def mask_and(a, b):
    return [x and y for x, y in zip(a, b)]


def mask_or(a, b):
    return [x or y for x, y in zip(a, b)]


def filter(df, mask):
    return df._select_rows_by_mask(list(mask))


def head(df, n=5):
    return df.head(n)


def set_index(df, name, drop: bool = True):
    """``drop=False`` keeps the column in the frame as well as using it for the row labels."""
    out = df.set_index(name)
    if not drop and not out.has_col(name):
        out[name] = list(df.col(name).values)
    return out


def reset_index(df, name=None):
    return df.reset_index(name)


def sort_values(df, by, ascending=True):
    return df.sort_values(by, ascending)


def df_label_where(df, col, pred: Callable, label_true, label_false):
    return [label_true if (not isna(v) and pred(v)) else label_false for v in df.col(col).values]


where = df_label_where


# ---- missing data -----------------------------------------------------------------------------------------
def dropna_any(df):
    keep = [all(not isna(c.values[i]) for c in df.columns) for i in range(df.nrows())]
    return df._select_rows_by_mask(keep)


def isna_count_by_col(df):
    return {c.name: sum(1 for v in c.values if isna(v)) for c in df.columns}


def fillna_value(df, col, value):
    d = df.copy()
    d[col] = [value if isna(v) else v for v in df.col(col).values]
    return d


def ffill(df, col, limit: int = None):
    """Carry the last present value forward; ``limit`` caps how many consecutive missing cells one value may fill
    (the reference's default is 1, legacy/src/momijo/dataframe/missing.mojo:560; here no limit unless given)."""
    out, last, run = [], None, 0
    for v in df.col(col).values:
        if not isna(v):
            last, run = v, 0
            out.append(v)
            continue
        run += 1
        out.append(last if (limit is None or run <= limit) else None)
    d = df.copy()
    d[col] = out
    return d


def interpolate_numeric(df, col):
    v = list(df.col(col).values)
    known = [i for i, x in enumerate(v) if not isna(x)]
    for a, b in zip(known, known[1:]):
        for i in range(a + 1, b):
            v[i] = v[a] + (v[b] - v[a]) * (i - a) / (b - a)
    d = df.copy()
    d[col] = v
    return d


def drop_duplicates(df, subset=None, keep: str = "first"):
    if keep != "first":
        return df.drop_duplicates(subset, keep)
    names = subset or df.col_names()
    seen, keep = set(), []
    for i in range(df.nrows()):
        k = tuple(df.col(n).values[i] for n in names)
        keep.append(k not in seen)
        seen.add(k)
    return df._select_rows_by_mask(keep)


# ---- statistics, rolling, ewm ---------------------------------------------------------------------------------
def col_mean(df, col):
    return Series(df.col(col).values).mean()


def compute_stats(values):
    s = Series(values)
    return {"count": s.count(), "mean": s.mean(), "std": s.std(), "min": s.min(), "max": s.max()}


def _roll(vals, window, fn):
    out = []
    for i in range(len(vals)):
        w = [v for v in vals[max(0, i - window + 1):i + 1] if not isna(v)]
        out.append(fn(w) if i + 1 >= window and len(w) == window else None)
    return out


def rolling_mean_f64(vals, window):
    return _roll(vals, window, lambda w: sum(w) / len(w))


def rolling_sum_f64(vals, window):
    return _roll(vals, window, sum)


def rolling_std_f64(vals, window, ddof=1):
    def f(w):
        if len(w) <= ddof:
            return None
        m = sum(w) / len(w)
        return math.sqrt(sum((v - m) ** 2 for v in w) / (len(w) - ddof))
    return _roll(vals, window, f)


def expanding_mean_f64(vals):
    out, s, n = [], 0.0, 0
    for v in vals:
        if not isna(v):
            s += v
            n += 1
        out.append(s / n if n else None)
    return out


def ewm_mean_f64(vals, alpha):
    out, m = [], None
    for v in vals:
        if isna(v):
            out.append(m)
            continue
        m = v if m is None else alpha * v + (1 - alpha) * m
        out.append(m)
    return out


def ewm_var_f64(vals, alpha):
    out, m, var = [], None, 0.0
    for v in vals:
        if isna(v):
            out.append(var if m is not None else None)
            continue
        if m is None:
            m, var = v, 0.0
        else:
            d = v - m
            m = m + alpha * d
            var = (1 - alpha) * (var + alpha * d * d)
        out.append(var)
    return out


def ewm_mean_f64_span(vals, span):
    return ewm_mean_f64(vals, 2.0 / (span + 1.0))


def ewm_var_f64_span(vals, span):
    return ewm_var_f64(vals, 2.0 / (span + 1.0))


# ---- groupby / pivot ----------------------------------------------------------------------------------------------
_AGG = {
    "sum": lambda x: sum(x), "mean": lambda x: sum(x) / len(x) if x else NaN, "min": lambda x: min(x) if x else NaN,
    "max": lambda x: max(x) if x else NaN, "count": lambda x: len(x), "first": lambda x: x[0] if x else None,
    "last": lambda x: x[-1] if x else None, "nunique": lambda x: len(set(x)),
    "std": lambda x: Series(x).std(), "median": lambda x: sorted(x)[len(x) // 2] if len(x) % 2 else
    (sum(sorted(x)[len(x) // 2 - 1:len(x) // 2 + 1]) / 2 if x else NaN),
}


class Agg:
    SUM, MEAN, MIN, MAX, COUNT = "sum", "mean", "min", "max", "count"

    def __init__(self, col: str, fn: str, out: Optional[str] = None):
        self.col, self.fn, self.out = col, fn, out or f"{col}_{fn}"

    # the spellings of ``AggSpec`` (relational.py), so that either record works with either group-by
    @property
    def column(self) -> str:
        return self.col

    @property
    def op(self) -> str:
        return self.fn

    @property
    def alias(self) -> str:
        return self.out

    def out_name(self) -> str:
        return self.out


def _groups(df, by):
    keys, order = {}, []
    for i in range(df.nrows()):
        k = tuple(df.col(b).values[i] for b in by)
        if k not in keys:
            keys[k] = []
            order.append(k)
        keys[k].append(i)
    return order, keys


def groupby(df, by, aggs) -> DataFrame:
    """``aggs``: {column: [fn, ...]} (reference signature) or a list of ``Agg``."""
    by = [by] if isinstance(by, str) else list(by)
    specs = aggs if isinstance(aggs, list) else [Agg(c, f) for c, fs in aggs.items() for f in fs]
    order, keys = _groups(df, by)
    out = {b: [k[j] for k in order] for j, b in enumerate(by)}
    for a in specs:
        vals = df.col(a.col).values
        out[a.out] = [_AGG[a.fn]([vals[i] for i in keys[k] if not isna(vals[i])]) for k in order]
    return DataFrame(out)


def groupby_transform(df, by, col, fn: str):
    by = [by] if isinstance(by, str) else list(by)
    order, keys = _groups(df, by)
    vals = df.col(col).values
    out = [None] * df.nrows()
    for k in order:
        r = _AGG[fn]([vals[i] for i in keys[k] if not isna(vals[i])])
        for i in keys[k]:
            out[i] = r
    return out


def pivot_table(df, index: str, columns: str, values: str, aggfunc: str = "mean", fill_value=None):
    rows_, cols_ = [], []
    for v in df.col(index).values:
        if v not in rows_:
            rows_.append(v)
    for v in df.col(columns).values:
        if v not in cols_:
            cols_.append(v)
    cells = {}
    for i in range(df.nrows()):
        v = df.col(values).values[i]
        if not isna(v):
            cells.setdefault((df.col(index).values[i], df.col(columns).values[i]), []).append(v)
    out = {index: rows_}
    for c in cols_:
        out[str(c)] = [_AGG[aggfunc](cells[(r, c)]) if (r, c) in cells else fill_value for r in rows_]
    return DataFrame(out)


# ---- joins --------------------------------------------------------------------------------------------------------
class Join:
    INNER, LEFT, RIGHT, OUTER = "inner", "left", "right", "outer"


class AsOf:
    BACKWARD, FORWARD, NEAREST = "backward", "forward", "nearest"


def merge(left, right, on, how: str = "inner", suffixes=("_x", "_y")):
    on = [on] if isinstance(on, str) else list(on)
    rkeys = {}
    for j in range(right.nrows()):
        rkeys.setdefault(tuple(right.col(k).values[j] for k in on), []).append(j)
    pairs, used = [], set()
    for i in range(left.nrows()):
        k = tuple(left.col(c).values[i] for c in on)
        js = rkeys.get(k, [])
        if js:
            for j in js:
                pairs.append((i, j))
                used.add(j)
        elif how in ("left", "outer"):
            pairs.append((i, None))
    if how in ("right", "outer"):
        pairs += [(None, j) for j in range(right.nrows()) if j not in used]
    if how == "right":
        pairs = [p for p in pairs if p[1] is not None]
    out = {}
    for k in on:
        out[k] = [left.col(k).values[i] if i is not None else right.col(k).values[j] for i, j in pairs]
    for c in left.columns:
        if c.name not in on:
            n = c.name + (suffixes[0] if right.has_col(c.name) else "")
            out[n] = [c.values[i] if i is not None else None for i, _ in pairs]
    for c in right.columns:
        if c.name not in on:
            n = c.name + (suffixes[1] if left.has_col(c.name) else "")
            out[n] = [c.values[j] if j is not None else None for _, j in pairs]
    return DataFrame(out)


def merge_asof(left, right, on, direction: str = "backward", tolerance=None):
    """Both frames sorted by ``on``; each left row takes the nearest right row in ``direction``."""
    rk = right.col(on).values
    out = left.to_dict()
    add = {c.name: [] for c in right.columns if c.name != on}
    for v in left.col(on).values:
        best = None
        for j, r in enumerate(rk):
            if isna(r) or isna(v):
                continue
            d = v - r
            ok = (direction == "backward" and d >= 0) or (direction == "forward" and d <= 0) or direction == "nearest"
            if ok and (tolerance is None or abs(d) <= tolerance):
                if best is None or abs(d) < abs(v - rk[best]) or (abs(d) == abs(v - rk[best]) and direction == "backward"):
                    best = j
        for n in add:
            add[n].append(right.col(n).values[best] if best is not None else None)
    for n, vals in add.items():
        out[n if n not in out else n + "_y"] = vals
    return DataFrame(out)


# ---- strings / datetime / categorical ---------------------------------------------------------------------------------
def _smap(df, col, fn):
    return [None if isna(v) else fn(str(v)) for v in df.col(col).values]


def str_title(df, col): return _smap(df, col, str.title)
def str_upper(df, col): return _smap(df, col, str.upper)
def str_lower(df, col): return _smap(df, col, str.lower)
def str_contains(df, col, pat, case_insensitive: bool = False, na_false: bool = True):
    """Per row, whether the cell contains ``pat``; missing cells give False, or None with ``na_false=False``
    (legacy/src/momijo/dataframe/string_ops.mojo:712-718)."""
    p = pat.lower() if case_insensitive else pat
    return [(False if na_false else None) if isna(v) else (p in (str(v).lower() if case_insensitive else str(v)))
            for v in df.col(col).values]
def str_slice(df, col, start, stop=None): return _smap(df, col, lambda s: s[start:stop])


def str_extract(df, col, pattern):
    def f(s):
        m = re.search(pattern, s)
        return (m.group(1) if m.groups() else m.group(0)) if m else None
    return _smap(df, col, f)


def str_replace_regex(df, col, pattern, repl):
    return _smap(df, col, lambda s: re.sub(pattern, repl, s))


def col_str_concat(df, a, b, sep=""):
    return [None if isna(x) or isna(y) else f"{x}{sep}{y}" for x, y in zip(df.col(a).values, df.col(b).values)]


def to_datetime(values):
    """ISO ``YYYY-MM-DD[ HH:MM:SS]`` strings -> (year, month, day, hour, minute, second) tuples."""
    out = []
    for v in values:
        m = re.match(r"(\d{4})-(\d{2})-(\d{2})(?:[ T](\d{2}):(\d{2})(?::(\d{2}))?)?", str(v)) if not isna(v) else None
        out.append(tuple(int(g) if g else 0 for g in m.groups()) if m else None)
    return out


def datetime_year(values, col: str = None, take: int = None):
    """Years of a list of date strings. The reference's frame form ``datetime_year(df, col, take=nrows)`` returns the
    first ``take`` cells of the column joined by ", " (cells shorter than four characters give an empty entry), or a
    warning text when the column is missing (legacy/src/momijo/dataframe/datetime_ops.mojo:116-150)."""
    if col is not None:
        if not values.has_col(col):
            return "[WARN] datetime_year: column not found"
        cells = ["" if isna(v) else str(v) for v in values.col(col).values]
        n = len(cells) if take is None else min(take, len(cells))
        return ", ".join(c if len(c) >= 4 else "" for c in cells[:n])
    return [None if d is None else d[0] for d in to_datetime(values)]


def datetime_year_df(df, col):
    return datetime_year(df.col(col).values)


def date_range(start: str, periods: int, freq_days: int = 1):
    import datetime as _dt

    d0 = _dt.date.fromisoformat(start)
    return [(d0 + _dt.timedelta(days=i * freq_days)).isoformat() for i in range(periods)]


def to_category(values, col_name: str = None, new_name: str = "category_code", ordered: bool = False, categories=()):
    """``to_category(values)`` -> (codes, categories sorted as text). The reference's frame form
    ``to_category(df, col_name, new_name, ordered, categories)`` returns a copy of the frame with an integer code column
    ``new_name``: categories in the given order (duplicates dropped) or in order of first appearance, -1 for values
    outside them; an unknown column leaves the frame unchanged (legacy/src/momijo/dataframe/categorical.mojo:210-290)."""
    if col_name is not None:
        out = values.copy()
        if not out.has_col(col_name):
            return out
        cells = ["" if isna(v) else str(v) for v in out.col(col_name).values]
        cats_f = []
        for v in (list(categories) if len(categories) else cells):
            if v not in cats_f:
                cats_f.append(v)
        pos = {c: i for i, c in enumerate(cats_f)}
        out[new_name] = [pos.get(v, -1) for v in cells]
        return out
    cats = []
    for v in values:
        if not isna(v) and v not in cats:
            cats.append(v)
    cats.sort(key=str)
    idx = {c: i for i, c in enumerate(cats)}
    return [idx[v] if not isna(v) else -1 for v in values], cats


# ---- I/O ------------------------------------------------------------------------------------------------------------------
def _parse(v):
    if v == "" or v is None:
        return None
    for cast in (int, float):
        try:
            return cast(v)
        except ValueError:
            pass
    return {"true": True, "false": False}.get(v.lower(), v)


def _csv_args(a, b, quotechar):
    """This package's order is (delimiter, header); the reference's is (header, delimiter, quotechar)
    (legacy/src/momijo/dataframe/io_csv.mojo:169-318). A bool in the first slot selects the reference's order."""
    if isinstance(a, bool):
        return (b if isinstance(b, str) else ","), a, quotechar
    return a, (b if isinstance(b, bool) else True), quotechar


def read_csv(path, delimiter=",", header=True, quotechar: str = '"'):
    delimiter, header, quotechar = _csv_args(delimiter, header, quotechar)
    with open(path, newline="") as f:
        rows_ = list(csv.reader(f, delimiter=delimiter, quotechar=quotechar))
    if not rows_:
        return DataFrame()
    names = rows_[0] if header else [f"c{i}" for i in range(len(rows_[0]))]
    body = rows_[1:] if header else rows_
    return DataFrame({n: [_parse(r[i]) if i < len(r) else None for r in body] for i, n in enumerate(names)})


def write_csv(df, path, delimiter=",", header=True, quotechar: str = '"'):
    delimiter, header, quotechar = _csv_args(delimiter, header, quotechar)
    with open(path, "w", newline="") as f:
        w = csv.writer(f, delimiter=delimiter, quotechar=quotechar)
        if header:
            w.writerow(df.col_names())
        for i in range(df.nrows()):
            w.writerow(["" if isna(c.values[i]) else c.values[i] for c in df.columns])
    return True


to_csv = write_csv


def read_json(path, lines=False):
    with open(path) as f:
        recs = [json.loads(l) for l in f if l.strip()] if lines else json.load(f)
    names = []
    for r in recs:
        for k in r:
            if k not in names:
                names.append(k)
    return DataFrame({n: [r.get(n) for r in recs] for n in names})


def write_json(df, path, lines=False):
    recs = [{k: (None if isna(v) else v) for k, v in r.items()} for r in df.to_records()]
    with open(path, "w") as f:
        if lines:
            for r in recs:
                f.write(json.dumps(r) + "\n")
        else:
            json.dump(recs, f)
    return True


to_json = write_json


def to_json_lines(df, path):
    return write_json(df, path, lines=True)


def read_json_lines(path):
    return read_json(path, lines=True)


class QueryExecutor:
    """Tiny query runner: ``select`` / ``where`` / ``order_by`` / ``limit`` over a frame
    (legacy/src/momijo/dataframe/exec.mojo:47)."""

    def __init__(self, df):
        self.df = df

    def where(self, col, op, value):
        import operator as o

        f = {"==": o.eq, "!=": o.ne, "<": o.lt, "<=": o.le, ">": o.gt, ">=": o.ge}[op]
        self.df = filter(self.df, [(not isna(v)) and f(v, value) for v in self.df.col(col).values])
        return self

    def select(self, *cols):
        self.df = select(self.df, cols)
        return self

    def order_by(self, col, ascending=True):
        self.df = self.df.sort_values(col, ascending)
        return self

    def limit(self, n):
        self.df = self.df.head(n)
        return self

    def collect(self):
        return self.df
