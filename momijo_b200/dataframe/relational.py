"""Joins, group-by, a small logical plan executor, expression predicates, resampling, categoricals, typed
series and the selection markers of the dataframe package under the reference's names
(legacy/src/momijo/dataframe/join.mojo, _groupby_core.mojo, exec.mojo, query.mojo, utils.mojo:294-710,
datetime_ops.mojo, categorical.mojo, series_*.mojo, selection.mojo)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .extras import coerce_to_f64, parse_f64_or_nan, try_parse_int_strict
from .frame import Bitmap, Column, DataFrame, NaN, Series, isna, string
from . import ops as _ops


# ---- joins -------------------------------------------------------------------------------------------------
def make_comp_key(df: DataFrame, cols: Sequence[str], row: int) -> str:
    """Composite key of a row: the cells of ``cols`` joined with the unit separator."""
    return "\x1f".join("" if isna(df.col(c).values[row]) else str(df.col(c).values[row]) for c in cols)


def _join(left, right, left_keys, right_keys, how, suffix_left="_x", suffix_right="_y"):
    lk, rk = list(left_keys), list(right_keys)
    index: Dict[str, List[int]] = {}
    for j in range(right.nrows()):
        index.setdefault(make_comp_key(right, rk, j), []).append(j)
    r_extra = [n for n in right.col_names() if n not in rk]
    clash = set(left.col_names()) & set(r_extra)
    lname = {n: (n + suffix_left if n in clash else n) for n in left.col_names()}
    rname = {n: (n + suffix_right if n in clash else n) for n in r_extra}
    out: Dict[str, List] = {lname[n]: [] for n in left.col_names()}
    out.update({rname[n]: [] for n in r_extra})
    used = set()

    def emit(i, j):
        for n in left.col_names():
            if i is not None:
                out[lname[n]].append(left.col(n).values[i])
            else:   # right-only row: the key columns take the right side's key values
                out[lname[n]].append(right.col(rk[lk.index(n)]).values[j] if n in lk else None)
        for n in r_extra:
            out[rname[n]].append(right.col(n).values[j] if j is not None else None)

    for i in range(left.nrows()):
        hits = index.get(make_comp_key(left, lk, i), [])
        if how == "anti":
            if not hits:
                emit(i, None)
            continue
        if hits:
            for j in hits:
                used.add(j)
                emit(i, j)
        elif how in ("left", "full"):
            emit(i, None)
    if how == "full":
        for j in range(right.nrows()):
            if j not in used:
                emit(None, j)
    if how == "anti":
        return DataFrame({n: out[lname[n]] for n in left.col_names()})
    return DataFrame(out)


def join_inner(left, right, left_keys, right_keys, suffix_left="_x", suffix_right="_y"):
    return _join(left, right, left_keys, right_keys, "inner", suffix_left, suffix_right)


def join_left(left, right, left_keys, right_keys, suffix_left="_x", suffix_right="_y"):
    return _join(left, right, left_keys, right_keys, "left", suffix_left, suffix_right)


def join_right(left, right, left_keys, right_keys, suffix_left="_x", suffix_right="_y"):
    """Every right row, with the left columns where a match exists (computed as a left join from the right)."""
    return _join(right, left, right_keys, left_keys, "left", suffix_right, suffix_left)


def join_full(left, right, left_keys, right_keys, suffix_left="_x", suffix_right="_y"):
    return _join(left, right, left_keys, right_keys, "full", suffix_left, suffix_right)


def join_anti(left, right, left_keys, right_keys):
    """Left rows without a match on the right."""
    return _join(left, right, left_keys, right_keys, "anti")


def inner_join(a, b, key_a: str, key_b: str): return join_inner(a, b, [key_a], [key_b])          # noqa: E704
def left_join_full(a, b, key_a: str, key_b: str): return join_left(a, b, [key_a], [key_b])      # noqa: E704
def right_join_full(a, b, key_a: str, key_b: str): return join_right(a, b, [key_a], [key_b])    # noqa: E704
def outer_join_full(a, b, key_a: str, key_b: str): return join_full(a, b, [key_a], [key_b])     # noqa: E704


def left_join(left, right, on):
    on = [on] if isinstance(on, str) else list(on)
    return join_left(left, right, on, on)


def asof_join(left: DataFrame, right: DataFrame, on: str, by: str = "") -> DataFrame:
    """For each left row the last right row with ``right[on] <= left[on]`` (within the same ``by`` value when
    given); unmatched rows get missing values in the right columns. Keys compare numerically when both parse
    as numbers, else as strings."""
    def key(v):
        f = parse_f64_or_nan(str(v))
        return (0, f) if f == f else (1, str(v))

    r_cols = [n for n in right.col_names() if n != on and n != by]
    out = {n: list(left.col(n).values) for n in left.col_names()}
    for n in r_cols:
        out[n + ("_y" if n in out else "")] = []
    names = [n + ("_y" if n in left.col_names() else "") for n in r_cols]
    order = sorted(range(right.nrows()), key=lambda j: key(right.col(on).values[j]))
    for i in range(left.nrows()):
        lv = key(left.col(on).values[i])
        best = None
        for j in order:
            if by and right.col(by).values[j] != left.col(by).values[i]:
                continue
            if key(right.col(on).values[j]) <= lv:
                best = j
            else:
                break
        for n, nm in zip(r_cols, names):
            out[nm].append(right.col(n).values[best] if best is not None else None)
    return DataFrame(out)


class ColMap:
    """Name -> output position."""

    def __init__(self):
        self.names: List[str] = []

    def add(self, name: str) -> int:
        self.names.append(name)
        return len(self.names) - 1

    def find(self, name: str) -> int:
        return self.names.index(name) if name in self.names else -1


class Acc:
    """Row accumulator used to build a join result column by column."""

    def __init__(self):
        self.names: List[str] = []
        self.cols: List[List] = []

    def add_schema(self, df: DataFrame, suffix: str = ""):
        for n in df.col_names():
            self.names.append(n + suffix)
            self.cols.append([])
        self._width = df.ncols()
        return self

    def append_row(self, df: DataFrame, row: int, valid_row: bool = True):
        base = len(self.cols) - df.ncols()
        for k, c in enumerate(df.columns):
            self.cols[base + k].append(c.values[row] if valid_row else None)
        return self


def materialize_two(accL: Acc, accR: Acc) -> DataFrame:
    out = {}
    for n, c in list(zip(accL.names, accL.cols)) + list(zip(accR.names, accR.cols)):
        out[n if n not in out else n + "_y"] = c
    return DataFrame(out)


def next_f64(): return [], [], False      # noqa: E704  (exhausted typed cursors of the reference's builder)
def next_i64(): return [], [], False      # noqa: E704
def next_bool(): return [], [], False     # noqa: E704
def next_str(): return [], [], False      # noqa: E704


# ---- group-by ------------------------------------------------------------------------------------------------
def apply_agg(values, func: str) -> Optional[float]:
    """sum / mean / min / max over the non-missing values; None when there are none."""
    clean = [float(v) for v in values if not isna(v)]
    if not clean:
        return None
    if func == "sum":
        return sum(clean)
    if func == "mean":
        return sum(clean) / len(clean)
    if func == "min":
        return min(clean)
    if func == "max":
        return max(clean)
    raise ValueError("Unsupported aggregation function")


def groupby_agg(df: DataFrame, by, aggs) -> DataFrame:
    """``aggs`` is a list of (column, function) pairs; result columns are named ``column_function``."""
    spec: Dict[str, List[str]] = {}
    for col, fn in aggs:
        spec.setdefault(col, []).append(fn)
    return _ops.groupby(df, by, spec)


def groupby_sum_f64(df: DataFrame, key: str, val: str) -> DataFrame:
    """(key, sum of val) in order of first appearance; cells that do not parse as numbers count as 0."""
    sums: Dict = {}
    for k, v in zip(df.col(key).values, df.col(val).values):
        f = coerce_to_f64(v)
        sums[k] = sums.get(k, 0.0) + (f if f == f else 0.0)
    return DataFrame({key: list(sums), val: list(sums.values())})


@dataclass
class AggSpec:
    column: str
    op: str = "sum"
    alias: str = ""

    def out_name(self) -> str:
        return self.alias or f"{self.column}_{self.op}"


def agg_on_col_rows(df: DataFrame, a: AggSpec, idxs) -> float:
    """sum / mean / count of a column over the given rows (missing cells skipped); unknown ops act as sum."""
    vals = [coerce_to_f64(df.col(a.column).values[i]) for i in idxs]
    vals = [v for v in vals if v == v]
    if a.op == "mean":
        return sum(vals) / len(vals) if vals else 0.0
    if a.op == "count":
        return float(len(vals))
    return float(sum(vals))


def agg_on_col(df: DataFrame, a: AggSpec) -> float:
    return agg_on_col_rows(df, a, range(df.nrows()))


def groupby_multi(df: DataFrame, keys, aggs) -> DataFrame:
    groups: Dict[str, List[int]] = {}
    for i in range(df.nrows()):
        groups.setdefault(make_comp_key(df, keys, i), []).append(i)
    out: Dict[str, List] = {k: [] for k in keys}
    for a in aggs:
        out[a.out_name()] = []
    for rows in groups.values():
        for k in keys:
            out[k].append(df.col(k).values[rows[0]])
        for a in aggs:
            out[a.out_name()].append(agg_on_col_rows(df, a, rows))
    return DataFrame(out)


def exec_aggregate(df: DataFrame, keys, aggs) -> DataFrame:
    if keys:
        return groupby_multi(df, keys, aggs)
    return DataFrame({a.out_name(): [agg_on_col(df, a)] for a in aggs})


# ---- predicates and the logical plan -------------------------------------------------------------------------------
class Ops:
    EQ, NE, LT, LE, GT, GE = 0, 1, 2, 3, 4, 5
    _text = {"==": 0, "=": 0, "!=": 1, "<>": 1, "<": 2, "<=": 3, ">": 4, ">=": 5}


class ExprKind:
    PRED, AND, OR, NOT = 0, 1, 2, 3


@dataclass
class ConstVal:
    is_num: bool = False
    num: float = 0.0
    text: str = ""


@dataclass
class Pred:
    column: str = ""
    op: int = Ops.EQ
    value: ConstVal = field(default_factory=ConstVal)


@dataclass
class Expr:
    kind: int = ExprKind.PRED
    pred: Optional[Pred] = None
    left: Optional["Expr"] = None
    right: Optional["Expr"] = None


def trim(s: str) -> str:
    return s.strip(" \t\r\n")


def sqrt64(x: float) -> float:
    return math.sqrt(x) if x > 0.0 else 0.0


def parse_op(tok: str) -> int:
    """Comparison operator code, -1 for anything else."""
    return Ops._text.get(tok, -1)


def parse_const(tok: str) -> ConstVal:
    t = trim(tok)
    if len(t) >= 2 and t[0] == t[-1] and t[0] in "'\"":
        return ConstVal(False, 0.0, t[1:-1])
    f = parse_f64_or_nan(t)
    return ConstVal(True, f, t) if f == f else ConstVal(False, 0.0, t)


def split_tokens(expr: str) -> List[str]:
    """Identifiers, numbers, quoted strings, comparison operators and the words and / or / not."""
    toks, i, n = [], 0, len(expr)
    while i < n:
        ch = expr[i]
        if ch.isspace():
            i += 1
        elif ch in "'\"":
            j = expr.find(ch, i + 1)
            j = n - 1 if j < 0 else j
            toks.append(expr[i:j + 1])
            i = j + 1
        elif expr[i:i + 2] in ("==", "!=", "<=", ">=", "<>"):
            toks.append(expr[i:i + 2])
            i += 2
        elif ch in "<>=()":
            toks.append(ch)
            i += 1
        else:
            j = i
            while j < n and not expr[j].isspace() and expr[j] not in "<>=!()'\"":
                j += 1
            toks.append(expr[i:j])
            i = max(j, i + 1)
    return toks


def parse_simple_expr(expr: str) -> Expr:
    """``col op const`` terms joined by ``and`` / ``or`` (left to right, ``and`` binds tighter), with ``not``
    in front of a term."""
    toks = split_tokens(expr)
    pos = 0

    def term() -> Expr:
        nonlocal pos
        if pos < len(toks) and toks[pos].lower() == "not":
            pos += 1
            return Expr(ExprKind.NOT, left=term())
        if pos < len(toks) and toks[pos] == "(":
            pos += 1
            e = disj()
            if pos < len(toks) and toks[pos] == ")":
                pos += 1
            return e
        col = toks[pos] if pos < len(toks) else ""
        op = parse_op(toks[pos + 1]) if pos + 1 < len(toks) else -1
        val = parse_const(toks[pos + 2]) if pos + 2 < len(toks) else ConstVal()
        pos += 3
        return Expr(ExprKind.PRED, Pred(col, op, val))

    def conj() -> Expr:
        nonlocal pos
        e = term()
        while pos < len(toks) and toks[pos].lower() == "and":
            pos += 1
            e = Expr(ExprKind.AND, left=e, right=term())
        return e

    def disj() -> Expr:
        nonlocal pos
        e = conj()
        while pos < len(toks) and toks[pos].lower() == "or":
            pos += 1
            e = Expr(ExprKind.OR, left=e, right=conj())
        return e

    return disj()


def eval_pred(df: DataFrame, p: Pred) -> Bitmap:
    out = Bitmap(df.nrows(), False)
    if not df.has_col(p.column) or p.op < 0:
        return out
    for i, v in enumerate(df.col(p.column).values):
        if isna(v):
            continue
        if p.value.is_num:
            a, b = coerce_to_f64(v), p.value.num
            if a != a:
                continue
        else:
            a, b = str(v), p.value.text
        out.set(i, [a == b, a != b, a < b, a <= b, a > b, a >= b][p.op])
    return out


def eval_expr(df: DataFrame, e: Expr) -> Bitmap:
    if e.kind == ExprKind.PRED:
        return eval_pred(df, e.pred)
    a = eval_expr(df, e.left)
    if e.kind == ExprKind.NOT:
        out = Bitmap(df.nrows(), False)
        out.bits = [not b for b in a.bits]
        return out
    b = eval_expr(df, e.right)
    out = Bitmap(df.nrows(), False)
    out.bits = [(x and y) if e.kind == ExprKind.AND else (x or y) for x, y in zip(a.bits, b.bits)]
    return out


def eval_where(df: DataFrame, expr_text: str) -> Bitmap:
    return eval_expr(df, parse_simple_expr(expr_text))


PLAN_SCAN, PLAN_FILTER, PLAN_PROJECT, PLAN_AGGREGATE, PLAN_SORT, PLAN_LIMIT = range(6)


@dataclass
class LogicalPlan:
    kind: int = PLAN_SCAN
    df: Optional[DataFrame] = None
    child: Optional["LogicalPlan"] = None
    expr: Optional[Expr] = None
    columns: List[str] = field(default_factory=list)
    group_keys: List[str] = field(default_factory=list)
    aggs: List[AggSpec] = field(default_factory=list)
    sort_keys: List[str] = field(default_factory=list)
    sort_asc: List[bool] = field(default_factory=list)
    limit: int = 0


def execute(plan: LogicalPlan) -> DataFrame:
    if plan.kind == PLAN_SCAN:
        return plan.df
    df = execute(plan.child)
    if plan.kind == PLAN_FILTER:
        return df._select_rows_by_mask(eval_expr(df, plan.expr).bits)
    if plan.kind == PLAN_PROJECT:
        return df._select_cols_by_names(plan.columns)
    if plan.kind == PLAN_AGGREGATE:
        return exec_aggregate(df, plan.group_keys, plan.aggs)
    if plan.kind == PLAN_SORT:
        return df.sort_values(plan.sort_keys, plan.sort_asc or True)
    if plan.kind == PLAN_LIMIT:
        return df.head(plan.limit)
    return df


def optimize_once(p: LogicalPlan) -> LogicalPlan:
    """One rewrite step: two stacked filters become one conjunction; a projection directly over a projection
    keeps only the outer column list."""
    if p.child is not None:
        p.child = optimize_once(p.child)
    if p.kind == PLAN_FILTER and p.child is not None and p.child.kind == PLAN_FILTER:
        return LogicalPlan(PLAN_FILTER, child=p.child.child, expr=Expr(ExprKind.AND, left=p.child.expr, right=p.expr))
    if p.kind == PLAN_PROJECT and p.child is not None and p.child.kind == PLAN_PROJECT:
        return LogicalPlan(PLAN_PROJECT, child=p.child.child, columns=p.columns)
    return p


def _plan_size(p: Optional[LogicalPlan]) -> int:
    return 0 if p is None else 1 + _plan_size(p.child)


def optimize(plan: LogicalPlan) -> LogicalPlan:
    """Apply ``optimize_once`` until the plan stops shrinking."""
    while True:
        n = _plan_size(plan)
        plan = optimize_once(plan)
        if _plan_size(plan) >= n:
            return plan


def query(df: DataFrame, expr: str) -> DataFrame:
    """``new = factor * col``, ``new = col * factor`` or ``new = col + bias``: a copy of the frame with the new
    column; anything else returns the frame unchanged (legacy/src/momijo/dataframe/query.mojo:110-228)."""
    if "=" not in expr:
        return df
    lhs, rhs = (trim(s) for s in expr.split("=", 1))
    for sym in ("*", "+"):
        if sym in rhs:
            a, b = (trim(s) for s in rhs.split(sym, 1))
            col, num = (a, b) if df.has_col(a) else (b, a)
            k = parse_f64_or_nan(num)
            if not df.has_col(col) or k != k:
                return df
            out = df.copy()
            src = [coerce_to_f64(v) for v in df.col(col).values]
            out[lhs] = [None if v != v else (v * k if sym == "*" else v + k) for v in src]
            return out
    return df


eval = query


def select_numeric(df: DataFrame) -> DataFrame:
    return df._select_cols_by_names([c.name for c in df.columns if c.dtype.name != "string"])


@dataclass
class Stats:
    count: int = 0
    mean: float = 0.0
    std: float = 0.0
    min: float = 0.0
    max: float = 0.0


# ---- datetime ---------------------------------------------------------------------------------------------------
def _pad2(n: int) -> str:
    return f"{n:02d}"


def parse_minutes(ts: str) -> int:
    """Minutes since midnight of a ``YYYY-MM-DD HH:MM[:SS]`` stamp; 0 when it does not have that shape."""
    if len(ts) < 16 or not (ts[11:13].isdigit() and ts[14:16].isdigit()):
        return 0
    return int(ts[11:13]) * 60 + int(ts[14:16])


def gen_dates_from(start_day: int, start_hour: int, start_min: int, n: int, step_min: int) -> List[str]:
    """``n`` stamps in January 2025 from the given day / hour / minute, ``step_min`` minutes apart."""
    total = start_day * 1440 + start_hour * 60 + start_min
    out = []
    for i in range(n):
        t = total + i * step_min
        out.append(f"2025-01-{_pad2(t // 1440)} {_pad2((t % 1440) // 60)}:{_pad2(t % 60)}:00")
    return out


def gen_dates_12h_from_2025_01_01(n: int) -> List[str]:
    return gen_dates_from(1, 0, 0, n, 720)


def tz_localize_utc(ts) -> List[str]:
    return [t + "+00:00" for t in ts]


def tz_convert(ts, target: str) -> List[str]:
    """Tags each stamp with the target zone (``stamp->zone``); no clock arithmetic, as in the reference."""
    return [f"{t}->{target}" for t in ts]


def _days_from_civil(y: int, m: int, d: int) -> int:
    y -= m <= 2
    era = (y if y >= 0 else y - 399) // 400
    yoe = y - era * 400
    doy = (153 * (m + (-3 if m > 2 else 9)) + 2) // 5 + d - 1
    return era * 146097 + yoe * 365 + yoe // 4 - yoe // 100 + doy - 719468


def _civil_from_days(z: int):
    z += 719468
    era = (z if z >= 0 else z - 146096) // 146097
    doe = z - era * 146097
    yoe = (doe - doe // 1460 + doe // 36524 - doe // 146096) // 365
    doy = doe - (365 * yoe + yoe // 4 - yoe // 100)
    mp = (5 * doy + 2) // 153
    d, m = doy - (153 * mp + 2) // 5 + 1, mp + (3 if mp < 10 else -9)
    return yoe + era * 400 + (m <= 2), m, d


class Resampler:
    """Down-sampling of a frame whose index holds ``YYYY-MM-DD[ HH:MM:SS]`` strings into bins of ``k`` days
    (``freq`` = ``"kD"``), anchored at the first date. Each aggregate returns a frame indexed by the bin's
    first day with one value per numeric column (non-numeric columns are left out)."""

    def __init__(self, base: DataFrame, freq: str):
        self.base, self.freq = base, freq
        t = freq.strip().upper()
        self.days = max(int(t[:-1] or 1), 1) if t.endswith("D") and (t[:-1].isdigit() or t[:-1] == "") else 1

    def _bins(self):
        days = []
        for lab in self.base.index.labels:
            s = str(lab)[:10]
            try:
                y, m, d = int(s[0:4]), int(s[5:7]), int(s[8:10])
                days.append(_days_from_civil(y, m, d))
            except ValueError:
                days.append(None)
        valid = [d for d in days if d is not None]
        if not valid:
            return {}, []
        d0 = min(valid)
        bins: Dict[int, List[int]] = {}
        for i, d in enumerate(days):
            if d is not None:
                bins.setdefault((d - d0) // self.days, []).append(i)
        keys = sorted(bins)
        labels = ["%04d-%02d-%02d" % _civil_from_days(d0 + k * self.days) for k in keys]
        return {k: bins[k] for k in keys}, labels

    def _agg(self, fn) -> DataFrame:
        bins, labels = self._bins()
        out = {}
        for c in self.base.columns:
            if c.dtype.name == "string":
                continue
            col = []
            for rows in bins.values():
                vals = [float(c.values[i]) for i in rows if not isna(c.values[i])]
                col.append(fn(vals) if vals else None)
            out[c.name] = col
        return DataFrame(out, index=labels)

    def sum(self, numeric_only: bool = True): return self._agg(sum)                              # noqa: E704
    def mean(self, numeric_only: bool = True): return self._agg(lambda v: sum(v) / len(v))       # noqa: E704
    def min(self, numeric_only: bool = True): return self._agg(min)                              # noqa: E704
    def max(self, numeric_only: bool = True): return self._agg(max)                              # noqa: E704

    def var(self, numeric_only: bool = True, ddof: int = 0):
        def f(v):
            if len(v) - ddof <= 0:
                return None
            m = sum(v) / len(v)
            return sum((x - m) ** 2 for x in v) / (len(v) - ddof)
        return self._agg(f)

    def std(self, numeric_only: bool = True, ddof: int = 0):
        d = self.var(numeric_only, ddof)
        for c in d.columns:
            c.values = [None if isna(v) else math.sqrt(v) for v in c.values]
        return d


def resample(df: DataFrame, freq: str) -> Resampler:
    return Resampler(df, freq)


# ---- categoricals and typed series ----------------------------------------------------------------------------------
class Categorical:
    """Values stored as codes into a list of categories (first-appearance order); missing values have code -1."""

    def __init__(self, values: Sequence = (), categories: Sequence = None):
        self._cats: List[str] = list(categories) if categories is not None else []
        self._codes: List[int] = []
        pos = {c: i for i, c in enumerate(self._cats)}
        for v in values:
            if isna(v) or v == "":
                self._codes.append(-1)
                continue
            if v not in pos:
                if categories is not None:
                    self._codes.append(-1)
                    continue
                pos[v] = len(self._cats)
                self._cats.append(v)
            self._codes.append(pos[v])

    def __len__(self):
        return len(self._codes)

    def __str__(self):
        return f"Categorical(n={len(self)}, categories={self._cats})"

    def get(self, i: int) -> str:
        c = self._codes[i] if 0 <= i < len(self._codes) else -1
        return self._cats[c] if c >= 0 else ""

    def categories(self) -> List[str]: return list(self._cats)       # noqa: E704
    def codes_list(self) -> List[int]: return list(self._codes)      # noqa: E704
    def unique(self) -> List[str]: return [self._cats[c] for c in dict.fromkeys(self._codes) if c >= 0]   # noqa: E704
    def values(self) -> List[str]: return [self.get(i) for i in range(len(self))]                          # noqa: E704

    def value_counts(self) -> Dict[str, int]:
        out = {c: 0 for c in self._cats}
        for c in self._codes:
            if c >= 0:
                out[self._cats[c]] += 1
        return out

    def astype(self, target: str) -> List[str]:
        return [str(c) for c in self._codes] if target in ("int", "codes") else self.values()

    def reorder(self, new_cats) -> "Categorical":
        """Same values under a new category list; values whose category is not listed become missing."""
        return Categorical(self.values(), list(new_cats))

    def remove_unused(self) -> "Categorical":
        used = {c for c in self._codes if c >= 0}
        return Categorical(self.values(), [c for i, c in enumerate(self._cats) if i in used])


def remove_unused(cat: Categorical) -> Categorical:
    return cat.remove_unused()


class _TypedSeries(Series):
    _conv = staticmethod(lambda v: v)

    def __init__(self, values=(), name: str = "", index=None, valid: Bitmap = None):
        vals = [None if isna(v) else self._conv(v) for v in values]
        if valid is not None:
            vals = [v if valid.get(i) else None for i, v in enumerate(vals)]
        super().__init__(vals, index, name)

    def get(self, i: int):
        return self.to_list()[i]

    def is_valid(self, i: int) -> bool:
        return not isna(self.to_list()[i])

    def len(self) -> int:
        return len(self)


class SeriesF64(_TypedSeries):
    _conv = staticmethod(float)


class SeriesI64(_TypedSeries):
    _conv = staticmethod(int)


class SeriesBool(_TypedSeries):
    _conv = staticmethod(bool)


class SeriesStr(_TypedSeries):
    _conv = staticmethod(str)


def get(s, i: int):
    """Element ``i`` of a series or column."""
    return s.get(i) if hasattr(s, "get") else s[i]


# ---- selection markers (legacy/src/momijo/dataframe/selection.mojo) ---------------------------------------------------
class RowAll:
    pass


class ColAll:
    pass


@dataclass
class PosSlice:
    start: int = 0
    stop: int = 0
    step: int = 1


ILocRowSlice = ILocColSlice = PosSlice


@dataclass
class LabelSlice:
    first: str = ""
    last: str = ""
    inclusive: bool = True


@dataclass
class RowPos:
    positions: List[int] = field(default_factory=list)


@dataclass
class Mask:
    bits: List[bool] = field(default_factory=list)


RowMask = Mask


class ColumnBoolOps:
    """Element-wise logic over boolean lists."""
    @staticmethod
    def and_(a, b): return [bool(x) and bool(y) for x, y in zip(a, b)]     # noqa: E704
    @staticmethod
    def or_(a, b): return [bool(x) or bool(y) for x, y in zip(a, b)]       # noqa: E704
    @staticmethod
    def not_(a): return [not bool(x) for x in a]                           # noqa: E704


def resolve_label_slice(index_labels, sel: LabelSlice) -> List[int]:
    """Positions covered by a label range; empty when either end is not in the index."""
    labs = [str(l) for l in index_labels]
    if sel.first not in labs or sel.last not in labs:
        return []
    a, b = labs.index(sel.first), labs.index(sel.last)
    if a > b:
        a, b = b, a
    return list(range(a, b + 1 if sel.inclusive else b))


def loc_impl_range(df: DataFrame, first, last) -> DataFrame:
    return df._select_rows_by_positions(resolve_label_slice(df.index.labels, LabelSlice(str(first), str(last))))


def loc_impl_indices(df: DataFrame, labels) -> DataFrame:
    labs = [str(l) for l in df.index.labels]
    return df._select_rows_by_positions([labs.index(str(l)) for l in labels if str(l) in labs])


def iloc_impl_indices_cols(df: DataFrame, rows, cols) -> DataFrame:
    d = df._select_cols_by_positions([c for c in cols if 0 <= c < df.ncols()])
    return d._select_rows_by_positions([r for r in rows if 0 <= r < df.nrows()])


# ---- small records -----------------------------------------------------------------------------------------------------
class ColKind:
    STR, I64, F64, BOOL = 0, 1, 2, 3


@dataclass
class ColPair:
    name: str = ""
    values: List = field(default_factory=list)
    kind: int = ColKind.STR


@dataclass
class IndexPair:
    pos: int = 0
    label: str = ""


def make_Index(n: int = 0) -> List[IndexPair]:
    return [IndexPair(i, str(i)) for i in range(max(n, 0))]


@dataclass
class ModuleState:
    keys: List[str] = field(default_factory=list)


def make_module_state(state=None) -> ModuleState:
    return ModuleState(list(state) if state else [])


class DTypesDoc:
    """Printable column -> dtype listing."""

    def __init__(self, df: DataFrame):
        self.rows = [(c.name, c.dtype.name) for c in df.columns]

    def __str__(self):
        return "\n".join(f"{n}: {t}" for n, t in self.rows)


class CellAccessor:
    """``acc[row, col_name]`` read / write access to a frame."""

    def __init__(self, df: DataFrame):
        self.df = df

    def __getitem__(self, key):
        r, c = key
        return self.df.col(c).values[r]

    def __setitem__(self, key, value):
        r, c = key
        self.df.col(c).values[r] = value


class ColNameList(list):
    """List of column names with membership helpers."""

    def index_of(self, name: str) -> int:
        return self.index(name) if name in self else -1


def sort_values_key(df: DataFrame, by: str, key) -> DataFrame:
    """Sort by ``key(cell)`` of column ``by`` (missing cells last)."""
    vals = df.col(by).values
    order = sorted(range(df.nrows()), key=lambda i: (isna(vals[i]), key(vals[i]) if not isna(vals[i]) else 0))
    return df._select_rows_by_positions(order)


def argsort_city_ts(df: DataFrame, city_col: str = "city", ts_col: str = "ts") -> List[int]:
    """Row order by (city, timestamp), both compared as strings."""
    c, t = df.col(city_col).values, df.col(ts_col).values
    return sorted(range(df.nrows()), key=lambda i: (str(c[i]), str(t[i])))


def rolling_mean(values, window: int):
    from .window import rolling_mean_f64
    return rolling_mean_f64(values, window)


def add_schema(acc: "Acc", df: DataFrame, suffix: str = "") -> None:
    """Function form of ``Acc.add_schema`` (the reference writes it at module level with the accumulator as its first
    argument, legacy/src/momijo/dataframe/join.mojo:140-171)."""
    acc.add_schema(df, suffix)


def append_row(acc: "Acc", df: DataFrame, row: int, valid_row: bool = True) -> None:
    """Function form of ``Acc.append_row`` (join.mojo:175-230)."""
    acc.append_row(df, row, valid_row)
