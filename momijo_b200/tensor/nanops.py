"""NaN-aware helpers (legacy/src/momijo/tensor/nanops.mojo:111-655)."""
import torch

from .tensor import _raw, _wrap


def isnan(x): return _wrap(torch.isnan(_raw(x)).to(torch.int64))
def isinf(x): return _wrap(torch.isinf(_raw(x)).to(torch.int64))
def isfinite(x): return _wrap(torch.isfinite(_raw(x)).to(torch.int64))


def nan_to_num(x, nan=0.0, posinf=None, neginf=None):
    return _wrap(torch.nan_to_num(_raw(x), nan=nan, posinf=posinf, neginf=neginf))


def nansum(x, axis=None, keepdims=False):
    return _wrap(torch.nansum(_raw(x)) if axis is None else torch.nansum(_raw(x), dim=axis, keepdim=keepdims))


def nanmean(x, axis=None, keepdims=False):
    return _wrap(torch.nanmean(_raw(x)) if axis is None else torch.nanmean(_raw(x), dim=axis, keepdim=keepdims))


def nanmin(x, axis=None, keepdims: bool = False):
    r = torch.where(torch.isnan(_raw(x)), torch.full_like(_raw(x), float("inf")), _raw(x))
    return _wrap(r.min() if axis is None else r.min(axis, keepdim=keepdims).values)


def nanmax(x, axis=None):
    r = torch.where(torch.isnan(_raw(x)), torch.full_like(_raw(x), float("-inf")), _raw(x))
    return _wrap(r.max() if axis is None else r.max(axis).values)


def nanstd(x, axis=None):
    r = _raw(x).double()
    m = torch.nanmean(r) if axis is None else torch.nanmean(r, dim=axis, keepdim=True)
    d = torch.where(torch.isnan(r), torch.zeros_like(r), (r - m) ** 2)
    n = (~torch.isnan(r)).sum() if axis is None else (~torch.isnan(r)).sum(axis)
    s = d.sum() if axis is None else d.sum(axis)
    return _wrap((s / n.clamp_min(1)).sqrt())


def safe_div(a, b, fill=0.0):
    from .math import safe_div as f

    return f(a, b, fill)


def safe_log(x, eps=1e-12):
    return _wrap(torch.log(_raw(x).double().clamp_min(eps)))


def safe_sqrt(x, eps: float = 0.0):
    """``sqrt(max(x, eps))`` element-wise (legacy/src/momijo/tensor/nanops.mojo:124-180)."""
    return _wrap(torch.sqrt(_raw(x).double().clamp_min(max(eps, 0.0))))


# ---- scalar and float64-specialised names (legacy/src/momijo/tensor/nanops.mojo:111-655) -----------------------------
import math as _math  # noqa: E402


def isnan_f64(v: float) -> bool: return v != v                          # noqa: E704
def isinf_f64(v: float) -> bool: return v in (_math.inf, -_math.inf)    # noqa: E704
def isfinite_f64(v: float) -> bool: return v == v and not isinf_f64(v)  # noqa: E704


def nan_to_num_f64(v: float, nan: float = 0.0, posinf: float = 1.7976931348623157e308,
                   neginf: float = -1.7976931348623157e308) -> float:
    return nan if v != v else (posinf if v == _math.inf else (neginf if v == -_math.inf else v))


def safe_log_scalar(x: float, eps: float = 1e-12) -> float:
    return _math.log(x if x > eps else eps)


def safe_sqrt_scalar(x: float, eps: float = 0.0) -> float:
    v = max(x, eps)
    return _math.sqrt(v) if v > 0 else 0.0


def nansum_all_f64(x) -> float: return float(torch.nansum(_raw(x).double()))            # noqa: E704
def nanmean_all_f64(x) -> float: return float(torch.nanmean(_raw(x).double()))          # noqa: E704


def nanmin_all_f64(x) -> float:
    r = _raw(x).double().reshape(-1)
    r = r[~torch.isnan(r)]
    return float(r.min()) if r.numel() else float("nan")


def _contig_args(x, a, b, c):
    """``f(x, axis)`` on a tensor, or the reference's ``f(data, shape, axis, keepdims)`` on a flat list."""
    if isinstance(a, (list, tuple)):
        return _wrap(torch.tensor(list(x), dtype=torch.float64).reshape(list(a))), b, bool(c)
    return x, a, False


def nansum_axis_contig_f64(x, axis=-1, ax=None, keepdims=False):       # noqa: E704
    t, a, k = _contig_args(x, axis, ax, keepdims)
    return nansum(t, a, k)


def nanmean_axis_contig_f64(x, axis=-1, ax=None, keepdims=False):      # noqa: E704
    t, a, k = _contig_args(x, axis, ax, keepdims)
    return nanmean(t, a, k)


def nanmin_axis_contig_f64(x, axis=-1, ax=None, keepdims=False):       # noqa: E704
    t, a, k = _contig_args(x, axis, ax, keepdims)
    return nanmin(t, a, k)


def safe_div_scalar(a: float, b: float, eps: float = 1e-12) -> float:
    """``a / b`` with a zero denominator replaced by ``eps`` (nanops.mojo:111-115)."""
    return a / (b if b != 0.0 else eps)
