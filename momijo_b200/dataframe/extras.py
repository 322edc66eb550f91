"""Smaller public helpers of the dataframe package under the reference's names: type tags and column
constructors (legacy/src/momijo/dataframe/api.mojo:144-230, 1310-1400, 2645-2830), list and printing helpers
(helpers.mojo:49-620), lenient parsers (compat.mojo:62-135), byte and text I/O (io_bytes.mojo, io_json_min.mojo,
io_csv.mojo, io_pickle_mnp.mojo), string helpers (string_ops.mojo), missing-value helpers (missing.mojo),
encoders (encoding.mojo) and the string / value-count statistics (stats_core.mojo)."""
from __future__ import annotations

import csv
import io
import json
import math
import os
from typing import Dict, List, Sequence

from .frame import (Bitmap, Column, DataFrame, DType, NaN, Series, bool_, float32, float64, int32, int64, isna,
                    string)


# ---- type tags --------------------------------------------------------------------------------------------
def tag_bool() -> int: return 1       # noqa: E704
def tag_int32() -> int: return 2      # noqa: E704
def tag_int64() -> int: return 3      # noqa: E704
def tag_float32() -> int: return 4    # noqa: E704
def tag_float64() -> int: return 5    # noqa: E704
def tag_string() -> int: return 6     # noqa: E704


_TAG_NAMES = {1: "bool", 2: "int32", 3: "int64", 4: "float32", 5: "float64", 6: "string"}
_DT_TAGS = {"bool": 1, "int32": 2, "int64": 3, "float32": 4, "float64": 5, "string": 6}


def tag_name(t: int) -> str:
    return _TAG_NAMES.get(t, "unknown")


dtype_name = tag_name


def dtype_to_tag(dt: DType) -> int:
    return _DT_TAGS.get(dt.name, 0)


def value_tag(v) -> int:
    """Tag of a cell (``Value`` or plain Python value); 0 for a missing one."""
    v = getattr(v, "v", v)
    if isna(v):
        return 0
    if isinstance(v, bool):
        return 1
    if isinstance(v, int):
        return 3
    if isinstance(v, float):
        return 5
    return 6


class ColumnTag:
    """Storage classes of a column: the 32-bit dtypes share the storage of their 64-bit siblings."""
    @staticmethod
    def F64() -> int: return 5     # noqa: E704
    @staticmethod
    def I64() -> int: return 3     # noqa: E704
    @staticmethod
    def STR() -> int: return 6     # noqa: E704
    @staticmethod
    def BOOL() -> int: return 1    # noqa: E704


def _storage_tag(c: Column) -> int:
    return {"float32": 5, "float64": 5, "int32": 3, "int64": 3, "bool": 1}.get(c.dtype.name, 6)


def is_f64_tag(tag: int) -> bool: return tag == ColumnTag.F64()      # noqa: E704
def is_i64_tag(tag: int) -> bool: return tag == ColumnTag.I64()      # noqa: E704
def is_str_tag(tag: int) -> bool: return tag == ColumnTag.STR()      # noqa: E704
def is_bool_tag(tag: int) -> bool: return tag == ColumnTag.BOOL()    # noqa: E704
def is_f64_col(c: Column) -> bool: return is_f64_tag(_storage_tag(c))    # noqa: E704
def is_i64_col(c: Column) -> bool: return is_i64_tag(_storage_tag(c))    # noqa: E704
def is_str_col(c: Column) -> bool: return is_str_tag(_storage_tag(c))    # noqa: E704
def is_bool_col(c: Column) -> bool: return is_bool_tag(_storage_tag(c))  # noqa: E704
def is_numeric_col(c: Column) -> bool: return _storage_tag(c) in (3, 5)  # noqa: E704


def dtype_name_of_column(c: Column) -> str:
    return c.dtype.name


def f64_nan() -> float:
    return NaN


def is_nan(x: float) -> bool:
    return x != x


# ---- parsers ------------------------------------------------------------------------------------------------
def try_parse_f64(s: str):
    """(value, ok): decimal or exponent notation with optional sign; surrounding blanks are ignored."""
    try:
        t = s.strip()
        if not t or t.lower() in ("nan", "inf", "+inf", "-inf", "infinity"):
            return 0.0, False
        return float(t), True
    except (ValueError, AttributeError):
        return 0.0, False


def parse_f64_or_nan(s: str) -> float:
    v, ok = try_parse_f64(s)
    return v if ok else NaN


def parse_f64(s: str, default: float = 0.0) -> float:
    v, ok = try_parse_f64(s)
    return v if ok else default


parse_f64_str = parse_f64


def parse_i64(s: str, default: int = 0) -> int:
    try:
        return int(s.strip())
    except (ValueError, AttributeError):
        return default


parse_i64_str = parse_i64


def atoi(s: str) -> int:
    """Leading optional sign and digits; anything after them is ignored, no digits give 0."""
    t, i, sign, v = s.strip(), 0, 1, 0
    if t[:1] in "+-" and t:
        sign, i = (-1 if t[0] == "-" else 1), 1
    while i < len(t) and t[i].isdigit():
        v = v * 10 + ord(t[i]) - 48
        i += 1
    return sign * v


def try_parse_int_strict(s: str):
    """(ok, value): the whole string must be an optionally signed run of digits."""
    t = s.strip()
    body = t[1:] if t[:1] in "+-" else t
    return (True, int(t)) if body.isdigit() else (False, 0)


def _norm_decimal(s: str) -> str:
    return s.replace(",", ".") if s.count(",") == 1 and "." not in s else s


def as_f64_or_nan(s: str) -> float:
    return parse_f64_or_nan(_norm_decimal(str(s).strip()))


def as_i64_or_zero(s: str) -> int:
    t = str(s).strip()
    ok, v = try_parse_int_strict(t)
    if ok:
        return v
    f = as_f64_or_nan(t)
    return int(f) if f == f and math.isfinite(f) else 0


def as_bool_or_false(s: str) -> bool:
    return str(s).strip().lower() in ("true", "1", "yes", "y", "on")


def as_str_or_empty(s) -> str:
    return "" if s is None else str(s)


def map_f64_or_nan(values): return [as_f64_or_nan(v) for v in values]         # noqa: E704
def map_i64_or_zero(values): return [as_i64_or_zero(v) for v in values]       # noqa: E704
def map_bool_or_false(values): return [as_bool_or_false(v) for v in values]   # noqa: E704
def map_str_or_empty(values): return [as_str_or_empty(v) for v in values]     # noqa: E704


def coerce_to_f64(v) -> float:
    return NaN if isna(v) else (as_f64_or_nan(v) if isinstance(v, str) else float(v))


def coerce_to_i64(v) -> int:
    return 0 if isna(v) else (as_i64_or_zero(v) if isinstance(v, str) else int(v))


def coerce_to_bool(v) -> bool:
    return False if isna(v) else (as_bool_or_false(v) if isinstance(v, str) else bool(v))


def is_digit(ch: str) -> bool: return len(ch) == 1 and "0" <= ch <= "9"                 # noqa: E704
def is_sign(ch: str) -> bool: return ch in ("+", "-")                                   # noqa: E704
def is_digit_like(ch: str) -> bool: return is_digit(ch) or ch in ("+", "-", ".")        # noqa: E704
def digit_value(ch: str) -> int: return ord(ch) - 48 if is_digit(ch) else -1            # noqa: E704
def digit_val(d: str) -> int: return max(digit_value(d), 0)                             # noqa: E704
def is_digit_code(c: int) -> bool: return 48 <= c <= 57                                 # noqa: E704
def is_alpha_code(c: int) -> bool: return 65 <= c <= 90 or 97 <= c <= 122               # noqa: E704
def is_space_code(c: int) -> bool: return c in (9, 10, 11, 12, 13, 32)                  # noqa: E704
def ascii_bytes(s: str) -> List[int]: return list(s.encode("latin-1", "replace"))       # noqa: E704
def ascii_at(s: str, i: int) -> int: return ord(s[i]) if 0 <= i < len(s) else 0         # noqa: E704
def code_at(s: str, i: int) -> int: return ascii_at(s, i)                               # noqa: E704
def min_int(a: int, b: int) -> int: return a if a < b else b                            # noqa: E704
def clamp(x, lo, hi): return lo if x < lo else (hi if x > hi else x)                    # noqa: E704


def infer_dtype(col) -> str:
    """"int", "float", "bool" or "string" for a list of strings or a ``Column`` (blank cells are skipped)."""
    vals = col.values if isinstance(col, Column) else list(col)
    cells = [str(v).strip() for v in vals if not isna(v) and str(v).strip() != ""]
    if not cells:
        return "string"
    if all(try_parse_int_strict(c)[0] for c in cells):
        return "int"
    if all(try_parse_f64(c)[1] for c in cells):
        return "float"
    if all(c.lower() in ("true", "false") for c in cells):
        return "bool"
    return "string"


# ---- list helpers -------------------------------------------------------------------------------------------------
def contains_string(xs, x) -> bool:
    return x in xs


def unique_strings_list(xs) -> List[str]:
    return list(dict.fromkeys(xs))


def list_union(a, b) -> List[str]:
    return list(dict.fromkeys(list(a) + list(b)))


union = list_union


def list_difference(a, b) -> List[str]:
    drop = set(b)
    return [x for x in dict.fromkeys(a) if x not in drop]


def symdiff(a, b) -> List[str]:
    return list_difference(a, b) + list_difference(b, a)


def between_i64(x: int, a: int, b: int) -> bool:
    return a <= x <= b


def take_i64(xs, idx): return [xs[i] for i in idx]     # noqa: E704


take_f64 = take_str = take_bool = take_i64


def isin_i64(xs, universe) -> List[bool]:
    u = set(universe)
    return [x in u for x in xs]


isin_f64 = isin_i64


def isin_string(s: str, universe) -> bool:
    return s in universe


def ge(col_vals, threshold: float) -> List[bool]:
    return [parse_f64_or_nan(str(v)) >= threshold for v in col_vals]


def isin(col_vals, values) -> List[bool]:
    u = set(values)
    return [v in u for v in col_vals]


def logical_and(a, b) -> List[bool]:
    return [bool(x) and bool(y) for x, y in zip(a, b)]


def between(col_vals, low: float, high: float, inclusive: bool = True) -> List[bool]:
    out = []
    for v in col_vals:
        x = parse_f64_or_nan(str(v))
        out.append((low <= x <= high) if inclusive else (low < x < high))
    return out


def find_first(xs, x) -> int:
    """Position of the first occurrence, -1 if absent."""
    try:
        return list(xs).index(x)
    except ValueError:
        return -1


def str_to(s: str) -> List[int]: return list(s.encode("utf-8"))                              # noqa: E704
def u32_to_le(x: int) -> List[int]: return list((x & 0xFFFFFFFF).to_bytes(4, "little"))     # noqa: E704
def u64_to_le(x: int) -> List[int]: return list((x & (2 ** 64 - 1)).to_bytes(8, "little"))  # noqa: E704
def i64_to_le(x: int) -> List[int]: return list(int(x).to_bytes(8, "little", signed=True))  # noqa: E704
def rep(s: str, n: int) -> str: return s * max(n, 0)                                        # noqa: E704
def pad(s: str, w: int) -> str: return s + " " * max(w - len(s), 0)                         # noqa: E704
def join_with(xs, sep: str) -> str: return sep.join(str(x) for x in xs)                     # noqa: E704
def join_i64_list(xs) -> str: return "[" + ", ".join(str(int(x)) for x in xs) + "]"         # noqa: E704
def join_f64_list(xs) -> str: return "[" + ", ".join(repr(float(x)) for x in xs) + "]"      # noqa: E704
def join_bool_list(xs) -> str: return "[" + ", ".join("True" if x else "False" for x in xs) + "]"   # noqa: E704
def to_string_list_i(xs) -> List[str]: return [str(int(x)) for x in xs]                     # noqa: E704
def to_string_list_f(xs) -> List[str]: return [repr(float(x)) for x in xs]                  # noqa: E704
def to_string_list_s(xs) -> List[str]: return [str(x) for x in xs]                          # noqa: E704


def range_str(start: int, stop: int, step: int = 1) -> List[str]:
    return [str(i) for i in range(start, stop, step or 1)]


def header(t: str) -> None:
    print(f"\n=== {t} ===")


def safe(op: str, ok: bool) -> None:
    print(f"[{'ok' if ok else 'FAIL'}] {op}")


def _head(label, xs, k, fmt):
    shown = ", ".join(fmt(x) for x in list(xs)[:max(k, 0)])
    print(f"{label}: [{shown}{', ...' if len(xs) > k else ''}] (n={len(xs)})")


def print_i64_head(label, xs, k): _head(label, xs, k, lambda x: str(int(x)))      # noqa: E704
def print_f64_head(label, xs, k): _head(label, xs, k, lambda x: repr(float(x)))   # noqa: E704
def print_str_head(label, xs, k): _head(label, xs, k, str)                        # noqa: E704


# ---- frame helpers ------------------------------------------------------------------------------------------------
def find_col(df: DataFrame, name: str) -> int:
    names = df.col_names()
    return names.index(name) if name in names else -1


col_index = find_col


def require_col_index(df: DataFrame, col: str) -> int:
    i = find_col(df, col)
    if i < 0:
        raise KeyError(f"column {col!r} not found")
    return i


def df_cell(df: DataFrame, c: int, r: int) -> str:
    v = df.columns[c].values[r]
    return "" if isna(v) else str(v)


def join_col_names(df: DataFrame) -> str:
    return ", ".join(df.col_names())


def print_df_info(df_name: str, df: DataFrame) -> None:
    print(f"{df_name}: {df.nrows()} rows x {df.ncols()} cols [{join_col_names(df)}]")


def print_df(df: DataFrame, rows: int = 5, mode: str = "head") -> None:
    part = df.tail(rows) if mode == "tail" else df.head(rows)
    print(repr(part))


show = print_df


def cols_by_name(df: DataFrame, names) -> List[Column]:
    return [df.col(n) for n in names]


def select_columns_safe(df: DataFrame, names) -> DataFrame:
    """Keep the requested columns that exist, in the requested order."""
    have = set(df.col_names())
    return df._select_cols_by_names([n for n in names if n in have])


def reorder(df: DataFrame, order) -> DataFrame:
    """Columns in ``order`` first (those that exist), the rest after them in their old order."""
    first = [n for n in order if df.has_col(n)]
    return df._select_cols_by_names(first + [n for n in df.col_names() if n not in first])


def equals(a: DataFrame, b: DataFrame) -> bool:
    if a.col_names() != b.col_names() or a.nrows() != b.nrows():
        return False
    for ca, cb in zip(a.columns, b.columns):
        for x, y in zip(ca.values, cb.values):
            if isna(x) != isna(y) or (not isna(x) and x != y):
                return False
    return True


def from_pairs(pairs) -> DataFrame:
    return DataFrame({name: list(values) for name, values in pairs})


def align_columns(left: DataFrame, right: DataFrame):
    """Both frames with the union of the column names (left's order, then right's extras); columns a side
    lacks are filled with missing values."""
    names = list_union(left.col_names(), right.col_names())

    def widen(df):
        return DataFrame({n: (list(df.col(n).values) if df.has_col(n) else [None] * df.nrows()) for n in names},
                         index=df.index.labels)
    return widen(left), widen(right)


def align_rows(left: DataFrame, right: DataFrame):
    """Both frames cut to the shorter one's number of rows."""
    n = min(left.nrows(), right.nrows())
    return left.head(n), right.head(n)


def df_head(df: DataFrame, n: int) -> DataFrame:
    return df.head(n)


def df_set_index(df: DataFrame, col_name: str) -> DataFrame:
    return df.set_index(col_name)


def df_reset_index(df: DataFrame) -> DataFrame:
    return df.reset_index()


def _numeric(df, col):
    return [coerce_to_f64(v) for v in df.col(col).values]


def df_nlargest(df: DataFrame, col: str, n: int) -> DataFrame:
    vals = _numeric(df, col)
    order = sorted((i for i in range(len(vals)) if vals[i] == vals[i]), key=lambda i: (-vals[i], i))
    return df._select_rows_by_positions(order[:max(n, 0)])


def df_nsmallest(df: DataFrame, col: str, n: int) -> DataFrame:
    vals = _numeric(df, col)
    order = sorted((i for i in range(len(vals)) if vals[i] == vals[i]), key=lambda i: (vals[i], i))
    return df._select_rows_by_positions(order[:max(n, 0)])


def df_clip(df: DataFrame, col: str, lo: float, hi: float) -> DataFrame:
    out = df.copy()
    out[col] = [v if isna(v) else min(max(v, lo), hi) for v in df.col(col).values]
    return out


def _fillna(df, col, fill):
    out = df.copy()
    out[col] = [fill if isna(v) else v for v in df.col(col).values]
    return out


df_fillna_i64 = df_fillna_f64 = df_fillna_bool = _fillna


def fillna_str_col(c: Column, fill: str) -> Column:
    return Column(c.name, [fill if isna(v) or v == "" else v for v in c.values], c.dtype)


def fillna_col_f64(c: Column, fill: float) -> Column:
    return Column(c.name, [fill if isna(v) else v for v in c.values], c.dtype)


fillna_col_bool = fillna_col_f64


def dropna_rows(df: DataFrame) -> DataFrame:
    """Rows without any missing cell (empty strings count as missing, as in the reference's string storage)."""
    keep = [i for i in range(df.nrows()) if not any(isna(c.values[i]) or c.values[i] == "" for c in df.columns)]
    return df._select_rows_by_positions(keep)


dropna_rows_any = dropna_rows


def drop_duplicates_rows(df: DataFrame, subset: str) -> DataFrame:
    seen, keep = set(), []
    for i, v in enumerate(df.col(subset).values):
        if v not in seen:
            seen.add(v)
            keep.append(i)
    return df._select_rows_by_positions(keep)


def df_where_qty_between(df: DataFrame, a: int, b: int) -> DataFrame:
    """Rows whose ``qty`` column lies in [a, b]."""
    vals = _numeric(df, "qty")
    return df._select_rows_by_positions([i for i, v in enumerate(vals) if v == v and a <= v <= b])


def filter_rows(df: DataFrame, mask) -> DataFrame:
    bits = mask.bits if isinstance(mask, Bitmap) else list(mask)
    return df._select_rows_by_positions([i for i, m in enumerate(bits) if m])


def labels_to_indices(index_labels, labels) -> List[int]:
    pos = {str(l): i for i, l in enumerate(index_labels)}
    return [pos[str(l)] for l in labels if str(l) in pos]


def labels_to_row_range(index_labels, first, last):
    """(start, stop) positions covering the inclusive label range; (0, 0) when a label is missing."""
    labs = [str(l) for l in index_labels]
    if str(first) not in labs or str(last) not in labs:
        return 0, 0
    a, b = labs.index(str(first)), labs.index(str(last))
    return (a, b + 1) if a <= b else (b, a + 1)


# ---- column constructors ------------------------------------------------------------------------------------
def _with_valid(name, data, valid, dtype):
    vals = list(data)
    if valid is not None:
        vals = [v if valid.get(i) else None for i, v in enumerate(vals)]
    return Column(name, vals, dtype)


def col_str(name, data): return Column(name, list(data), string)                                     # noqa: E704
def col_string(name, data, valid: Bitmap = None): return _with_valid(name, data, valid, string)     # noqa: E704
def col_f64(name, data, valid: Bitmap = None): return _with_valid(name, data, valid, float64)       # noqa: E704
def col_i64(name, data, valid: Bitmap = None): return _with_valid(name, data, valid, int64)         # noqa: E704
def col_bool(name, data, valid: Bitmap = None): return _with_valid(name, data, valid, bool_)        # noqa: E704


col_string_with_valid, col_f64_with_valid = col_string, col_f64
col_i64_with_valid, col_bool_with_valid = col_i64, col_bool


def col_from_list(name, values) -> Column:
    return Column(name, list(values))


def from_list_int(name, values) -> Column:
    return Column(name, [int(v) for v in values], int64)


def is_valid_cell(c: Column, i: int) -> bool:
    return 0 <= i < len(c) and not isna(c.values[i])


def set_cell_preserve_type(c: Column, i: int, value) -> Column:
    """Copy of the column with cell ``i`` replaced; the value is converted to the column's type."""
    out = c.copy()
    tag = _storage_tag(c)
    out.values[i] = None if isna(value) else (coerce_to_f64(value) if tag == 5 else coerce_to_i64(value) if tag == 3
                                              else coerce_to_bool(value) if tag == 1 else str(value))
    return out


def rebuild_column_with(c: Column, values) -> Column:
    return Column(c.name, list(values), c.dtype)


def make_bitmap(n: int, fill: bool = True) -> Bitmap:
    return Bitmap(n, fill)


def coerce_str_to_i64(df: DataFrame, col: str) -> DataFrame:
    out = df.copy()
    out[col] = Column(col, [None if isna(v) or str(v).strip() == "" else as_i64_or_zero(v) for v in df.col(col).values],
                      int64)
    return out


def series_values(s: Series) -> str:
    return "[" + ", ".join(str(v) for v in s.to_list()) + "]"


def resample_sum_min(series, freq: int) -> List[float]:
    """Sums over consecutive groups of ``freq`` samples (the last group may be short)."""
    f = max(freq, 1)
    return [float(sum(series[i:i + f])) for i in range(0, len(series), f)]


# ---- strings ---------------------------------------------------------------------------------------------------
def str_split_once(s: str, sep: str):
    """(before, after) around the first ``sep``; (s, "") when it does not occur."""
    i = s.find(sep) if sep else -1
    return (s, "") if i < 0 else (s[:i], s[i + len(sep):])


def str_strip(s: str) -> str:
    return s.strip(" \t\r\n")


def compare_str_eq(a, b) -> List[int]:
    return [1 if x == y else 0 for x, y in zip(a, b)]


def contains_digit(s: str) -> bool:
    return any("0" <= ch <= "9" for ch in s)


def extract_first_alpha(s: str) -> str:
    """First maximal run of ASCII letters."""
    out = ""
    for ch in s:
        if is_alpha_code(ord(ch)):
            out += ch
        elif out:
            break
    return out


def extract_all_alpha_joined(s: str) -> str:
    return "".join(ch for ch in s if is_alpha_code(ord(ch)))


def split_on_delims(s: str) -> List[str]:
    """Split on blanks, commas, semicolons and pipes; empty pieces are dropped."""
    out, cur = [], ""
    for ch in s:
        if ch in " \t\r\n,;|":
            if cur:
                out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur:
        out.append(cur)
    return out


def rpad(s: str, width: int, fill: str = " ") -> str:
    f = fill[:1] or " "
    return s + f * max(width - len(s), 0)


def str_len(df: DataFrame, col: str) -> List[float]:
    return [NaN if isna(v) else float(len(str(v))) for v in df.col(col).values]


def str_contains_s(s: str, sub: str) -> bool:
    return sub in s


def str_replace_all(s: str, old: str, newv: str) -> str:
    return s.replace(old, newv) if old else s


def value_counts_str(xs) -> DataFrame:
    """Frame of (value, count), most frequent first, ties by first appearance."""
    counts: Dict[str, int] = {}
    for x in xs:
        counts[x] = counts.get(x, 0) + 1
    order = sorted(counts, key=lambda k: (-counts[k], list(counts).index(k)))
    return DataFrame({"value": order, "count": [counts[k] for k in order]})


def value_counts_bins(xs, bins: int) -> DataFrame:
    """Counts over ``bins`` equal-width intervals of [min, max]; columns ``bin`` ("lo-hi") and ``count``."""
    vals = [x for x in xs if not isna(x)]
    if not vals or bins <= 0:
        return DataFrame({"bin": [], "count": []})
    lo, hi = min(vals), max(vals)
    width = (hi - lo) / bins or 1.0
    counts = [0] * bins
    for v in vals:
        counts[min(int((v - lo) / width), bins - 1)] += 1
    labels = [f"{lo + i * width:g}-{lo + (i + 1) * width:g}" for i in range(bins)]
    return DataFrame({"bin": labels, "count": counts})


def get_dummies_str(df: DataFrame, col: str, drop_first: bool = False, prefix: str = "") -> DataFrame:
    """One 0/1 column per distinct value of ``col`` (first-appearance order), named ``prefix_value``; the source
    column is dropped."""
    vals = df.col(col).values
    cats = [c for c in dict.fromkeys(vals) if not isna(c)]
    if drop_first:
        cats = cats[1:]
    out = df.drop(col)
    p = prefix or col
    for c in cats:
        out[f"{p}_{c}"] = [1 if v == c else 0 for v in vals]
    return out


# ---- bytes and text ---------------------------------------------------------------------------------------------
def str_to_bytes(s: str) -> List[int]: return list(s.encode("utf-8"))       # noqa: E704


string_to_bytes = str_to_bytes


def ascii_byte_to_string(v: int) -> str:
    return chr(v) if 0 <= v < 128 else "?"


def u8_to_char(b: int) -> str:
    return chr(int(b) & 255)


def bytes_to_string(b) -> str:
    return bytes(b).decode("utf-8", "replace")


def write_bytes(path: str, data) -> bool:
    try:
        with open(path, "wb") as f:
            f.write(bytes(data))
        return True
    except OSError:
        return False


def read_bytes(path: str) -> List[int]:
    try:
        with open(path, "rb") as f:
            return list(f.read())
    except OSError:
        return []


def write_text(path: str, text: str) -> bool:
    try:
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        with open(path, "w") as f:
            f.write(text)
        return True
    except OSError:
        return False


def read_text(path: str) -> str:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return ""


def json_escape(s: str) -> str:
    return json.dumps(s)[1:-1]


def json_unescape(s: str) -> str:
    try:
        return json.loads('"' + s + '"')
    except ValueError:
        return s


def json_field(obj_text: str, key: str) -> str:
    """Value of ``key`` in a JSON object given as text, as a string ("" if absent or not an object)."""
    try:
        v = json.loads(obj_text).get(key, "")
    except (ValueError, AttributeError):
        return ""
    return v if isinstance(v, str) else json.dumps(v)


def _records(df):
    return [{k: (None if isna(v) else v) for k, v in r.items()} for r in df.to_records()]


def _from_records(recs) -> DataFrame:
    names: List[str] = []
    for r in recs:
        for k in r:
            if k not in names:
                names.append(k)
    return DataFrame({n: [r.get(n) for r in recs] for n in names})


def to_json_string(df: DataFrame) -> str:
    return json.dumps(_records(df))


def from_json_string(s: str) -> DataFrame:
    try:
        recs = json.loads(s)
    except ValueError:
        return DataFrame()
    return _from_records(recs if isinstance(recs, list) else [recs])


def to_json_lines_string(df: DataFrame) -> str:
    return "".join(json.dumps(r) + "\n" for r in _records(df))


def from_json_lines_string(s: str) -> DataFrame:
    recs = []
    for line in s.splitlines():
        if line.strip():
            try:
                recs.append(json.loads(line))
            except ValueError:
                continue
    return _from_records(recs)


def to_csv_string(df: DataFrame, delimiter=",", header=True, quotechar: str = '"') -> str:
    """``to_csv_string(df, delimiter, header)``, or the reference's ``(df, header, delimiter, quotechar)``: a bool in
    the first slot selects its order (legacy/src/momijo/dataframe/io_csv.mojo:169-174)."""
    if isinstance(delimiter, bool):
        delimiter, header = (header if isinstance(header, str) else ","), delimiter
    buf = io.StringIO()
    w = csv.writer(buf, delimiter=delimiter, lineterminator="\n", quotechar=quotechar)
    if header:
        w.writerow(df.col_names())
    for i in range(df.nrows()):
        w.writerow(["" if isna(c.values[i]) else c.values[i] for c in df.columns])
    return buf.getvalue()


def read_csv_from_string(text: str, delimiter: str = ",", header: bool = True, quote: str = '"') -> DataFrame:
    from .ops import _parse
    rows = list(csv.reader(io.StringIO(text), delimiter=delimiter, quotechar=quote))
    rows = [r for r in rows if r]
    if not rows:
        return DataFrame()
    names = rows[0] if header else [f"c{i}" for i in range(len(rows[0]))]
    body = rows[1:] if header else rows
    return DataFrame({n: [_parse(r[i]) if i < len(r) else None for r in body] for i, n in enumerate(names)})


def read_csv_string(text: str, delimiter: str = ",", header: bool = True, usecols=None, dtypes: Dict[str, str] = None):
    df = read_csv_from_string(text, delimiter, header)
    if usecols:
        df = select_columns_safe(df, usecols)
    if dtypes:
        from .ops import astype
        for col, dt in dtypes.items():
            if df.has_col(col):
                df = astype(df, col, dt)
    return df


def _esc(s: str) -> str:
    return s.replace("\\", "\\\\").replace("\t", "\\t").replace("\n", "\\n").replace("\r", "\\r")


def _unesc(s: str) -> str:
    out, i = "", 0
    while i < len(s):
        if s[i] == "\\" and i + 1 < len(s):
            out += {"t": "\t", "n": "\n", "r": "\r", "\\": "\\"}.get(s[i + 1], s[i + 1])
            i += 2
        else:
            out += s[i]
            i += 1
    return out


def to_mnp_string(df: DataFrame) -> str:
    """Text form of a frame: ``MNP``, ``nrows<TAB>ncols``, the index name, the column names, then one line per
    row; tabs, newlines and backslashes inside cells are backslash-escaped (missing cells are empty)."""
    lines = ["MNP", f"{df.nrows()}\t{df.ncols()}", _esc(getattr(df, "index_name", "") or ""),
             "\t".join(_esc(n) for n in df.col_names())]
    for i in range(df.nrows()):
        lines.append("\t".join("" if isna(c.values[i]) else _esc(str(c.values[i])) for c in df.columns))
    return "\n".join(lines) + "\n"


def from_mnp_string(s: str) -> DataFrame:
    from .ops import _parse
    lines = s.split("\n")
    if len(lines) < 4 or not lines[0].startswith("MNP"):
        return DataFrame()
    try:
        nrows, ncols = (int(v) for v in lines[1].split("\t"))
    except ValueError:
        return DataFrame()
    names = [_unesc(n) for n in lines[3].split("\t")] if ncols else []
    cols: List[List] = [[] for _ in names]
    for line in lines[4:4 + nrows]:
        cells = line.split("\t")
        for j in range(len(names)):
            cols[j].append(_parse(_unesc(cells[j])) if j < len(cells) else None)
    df = DataFrame(dict(zip(names, cols)))
    df.index_name = _unesc(lines[2])
    return df
