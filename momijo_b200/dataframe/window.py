"""Rolling, expanding and exponentially weighted statistics over plain lists
(legacy/src/momijo/dataframe/utils.mojo:921-1760).

Rolling functions return ``None`` until a full window is available; variances default to the population
form (``ddof=0``) and give ``None`` when ``window - ddof <= 0``. Exponentially weighted functions follow
the recursive form by default and the weight-normalised one with ``adjust=True``; an ``alpha`` outside
(0, 1] gives an empty list. ``*_int`` names take integers and are the same computation."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence


def _rolling(values: Sequence, window: int, fn) -> List:
    n = len(values)
    if window <= 0 or n == 0:
        return []
    return [None if i + 1 < window else fn(values[i + 1 - window:i + 1]) for i in range(n)]


def rolling_sum_f64(values, window): return _rolling(values, window, lambda w: float(sum(w)))          # noqa: E704
def rolling_sum_int(values, window): return _rolling(values, window, lambda w: int(sum(w)))            # noqa: E704
def rolling_mean_f64(values, window): return _rolling(values, window, lambda w: sum(w) / len(w))       # noqa: E704
def rolling_min_f64(values, window): return _rolling(values, window, min)                               # noqa: E704
def rolling_max_f64(values, window): return _rolling(values, window, max)                               # noqa: E704


rolling_sum = rolling_sum_f64
rolling_mean_int = rolling_mean_f64
rolling_min_int = rolling_min_f64
rolling_max_int = rolling_max_f64


def rolling_var_f64(values, window: int, ddof: int = 0):
    def var(w):
        cnt = len(w)
        if cnt - ddof <= 0:
            return None
        m = sum(w) / cnt
        v = sum(x * x for x in w) / cnt - m * m
        if ddof:
            v = v * cnt / (cnt - ddof)
        return max(v, 0.0)
    return _rolling(values, window, var)


def rolling_std_f64(values, window: int, ddof: int = 0):
    return [None if v is None else math.sqrt(v) for v in rolling_var_f64(values, window, ddof)]


rolling_var_int, rolling_std_int = rolling_var_f64, rolling_std_f64


def rolling_abs(values, window: int):
    """Rolling mean of absolute values."""
    return _rolling([abs(v) for v in values], window, lambda w: sum(w) / len(w))


# ---- expanding ----------------------------------------------------------------------------------------------
def expanding_sum_f64(values):
    out, s = [], 0.0
    for v in values:
        s += v
        out.append(s)
    return out


def expanding_sum_int(values):
    return [int(v) for v in expanding_sum_f64(values)]


def expanding_mean_f64(values, min_periods: int = 1):
    """NaN until ``min_periods`` observations have been seen."""
    out, s = [], 0.0
    for i, v in enumerate(values):
        s += v
        out.append(s / (i + 1) if i + 1 >= max(min_periods, 1) else float("nan"))
    return out


expanding_mean_int = expanding_mean_f64


def expanding_abs_mean_f64(values):
    return expanding_mean_f64([abs(v) for v in values])


expanding_abs_mean_int = expanding_abs_mean_f64


def _running(values, pick):
    out, cur = [], None
    for v in values:
        cur = v if cur is None else pick(cur, v)
        out.append(cur)
    return out


def expanding_min_f64(values): return _running(values, min)     # noqa: E704
def expanding_max_f64(values): return _running(values, max)     # noqa: E704


expanding_min_int, expanding_max_int = expanding_min_f64, expanding_max_f64


def expanding_var_f64(values, ddof: int = 0):
    """Variance of the first i+1 values; NaN while ``i + 1 - ddof <= 0``."""
    out, s1, s2 = [], 0.0, 0.0
    for i, v in enumerate(values):
        s1 += v
        s2 += v * v
        cnt = i + 1
        if cnt - ddof <= 0:
            out.append(float("nan"))
            continue
        m = s1 / cnt
        var = s2 / cnt - m * m
        if ddof:
            var = var * cnt / (cnt - ddof)
        out.append(max(var, 0.0))
    return out


def expanding_std_f64(values, ddof: int = 0):
    return [math.sqrt(v) if v == v else v for v in expanding_var_f64(values, ddof)]


expanding_var_int, expanding_std_int = expanding_var_f64, expanding_std_f64


def cum_sum(values):
    return expanding_sum_f64(values)


def cum_mean(values):
    return expanding_mean_f64(values)


# ---- exponentially weighted -------------------------------------------------------------------------------------
def _alpha_from_span(span: int) -> float:
    return 2.0 / (float(max(span, 1)) + 1.0)


def ewm_mean_f64(values, alpha: float, adjust: bool = False) -> List[float]:
    n = len(values)
    if n == 0 or alpha <= 0.0 or alpha > 1.0:
        return []
    if not adjust:
        out, y = [float(values[0])], float(values[0])
        for v in values[1:]:
            y = (1.0 - alpha) * y + alpha * v
            out.append(y)
        return out
    num, den = alpha * values[0], alpha
    out = [num / den]
    for v in values[1:]:
        num = (1.0 - alpha) * num + alpha * v
        den = (1.0 - alpha) * den + alpha
        out.append(num / den)
    return out


def ewm_var_f64(values, alpha: float, adjust: bool = False) -> List[float]:
    n = len(values)
    if n == 0 or alpha <= 0.0 or alpha > 1.0:
        return []
    out = [0.0]
    if not adjust:
        m, v = float(values[0]), 0.0
        for x in values[1:]:
            dm = x - m
            m += alpha * dm
            v = max((1.0 - alpha) * (v + alpha * dm * dm), 0.0)
            out.append(v)
        return out
    num_m, den_m = alpha * values[0], alpha
    mean, num_c, den_c = num_m / den_m, 0.0, 0.0
    for x in values[1:]:
        num_m = (1.0 - alpha) * num_m + alpha * x
        den_m = (1.0 - alpha) * den_m + alpha
        prev, mean = mean, num_m / den_m
        dx = x - prev
        num_c = (1.0 - alpha) * num_c + alpha * dx * dx
        den_c = (1.0 - alpha) * den_c + alpha
        out.append(max(num_c / den_c, 0.0) if den_c > 0.0 else 0.0)
    return out


def ewm_std_f64(values, alpha: float, adjust: bool = False) -> List[float]:
    return [math.sqrt(v) for v in ewm_var_f64(values, alpha, adjust)]


ewm_mean_int, ewm_var_int, ewm_std_int = ewm_mean_f64, ewm_var_f64, ewm_std_f64


def ewm_mean_f64_span(values, span: int, adjust: bool = False): return ewm_mean_f64(values, _alpha_from_span(span), adjust)   # noqa: E704,E501
def ewm_var_f64_span(values, span: int, adjust: bool = False): return ewm_var_f64(values, _alpha_from_span(span), adjust)     # noqa: E704,E501
def ewm_std_f64_span(values, span: int, adjust: bool = False): return ewm_std_f64(values, _alpha_from_span(span), adjust)     # noqa: E704,E501


ewm_mean_int_span, ewm_var_int_span, ewm_std_int_span = ewm_mean_f64_span, ewm_var_f64_span, ewm_std_f64_span


def exp_f64(values) -> List[float]:
    return [math.exp(v) for v in values]


exp_int = exp_f64


# ---- shifts and ranks (legacy/src/momijo/dataframe/frame.mojo: lag, lead, row_number, dense_rank) ---------------
def lag(values, k: int = 1, fill=None) -> List:
    k = max(k, 0)
    return [fill] * min(k, len(values)) + list(values[:max(len(values) - k, 0)])


def lead(values, k: int = 1, fill=None) -> List:
    k = max(k, 0)
    return list(values[k:]) + [fill] * min(k, len(values))


def row_number(n_or_values) -> List[int]:
    n = n_or_values if isinstance(n_or_values, int) else len(n_or_values)
    return list(range(1, n + 1))


def rank_dense_f64(xs) -> List[int]:
    """Dense rank starting at 1 (equal values share a rank, ranks have no gaps)."""
    order = {v: i + 1 for i, v in enumerate(sorted(set(xs)))}
    return [order[v] for v in xs]


dense_rank = rank_dense_f64


def percentile_f64(xs, p: float) -> float:
    """Linear-interpolation percentile, ``p`` in [0, 100]; NaN for an empty list."""
    if not xs:
        return float("nan")
    s = sorted(xs)
    pos = (len(s) - 1) * min(max(p, 0.0), 100.0) / 100.0
    lo = int(math.floor(pos))
    hi = min(lo + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (pos - lo)


def nlargest_f64(xs, n: int) -> List[int]:
    """Indices of the ``n`` largest values, largest first (ties by position)."""
    return sorted(range(len(xs)), key=lambda i: (-xs[i], i))[:max(n, 0)]


def nsmallest_f64(xs, n: int) -> List[int]:
    return sorted(range(len(xs)), key=lambda i: (xs[i], i))[:max(n, 0)]


def clip_f64(xs, lo: float, hi: float) -> List[float]:
    return [min(max(x, lo), hi) for x in xs]


def corr_f64(x, y) -> float:
    """Pearson correlation; 0.0 when either side has no variance or the lengths differ."""
    n = len(x)
    if n == 0 or n != len(y):
        return 0.0
    mx, my = sum(x) / n, sum(y) / n
    sxx = sum((a - mx) ** 2 for a in x)
    syy = sum((b - my) ** 2 for b in y)
    if sxx <= 0.0 or syy <= 0.0:
        return 0.0
    return sum((a - mx) * (b - my) for a, b in zip(x, y)) / math.sqrt(sxx * syy)


corr = corr_f64


def cumsum_i64(xs) -> List[int]:
    return expanding_sum_int(xs)


def sqrt_f64(x: float) -> float:
    return math.sqrt(x) if x > 0.0 else 0.0


def searchsorted_f64(sorted_xs, x: float) -> int:
    """First position whose value is >= x (left insertion point)."""
    import bisect
    return bisect.bisect_left(sorted_xs, x)


def argsort_f64(xs, asc: bool = True) -> List[int]:
    """Stable argsort."""
    return sorted(range(len(xs)), key=lambda i: xs[i], reverse=not asc) if asc else \
        sorted(range(len(xs)), key=lambda i: (-xs[i], i))


argsort_i64 = argsort_f64
