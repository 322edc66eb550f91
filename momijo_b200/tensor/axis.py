"""Axis utilities and reductions (legacy/src/momijo/tensor/axis.mojo:128-1294)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .tensor import _raw, _wrap


def moveaxis(x, src: int, dst: int):
    return _wrap(torch.movedim(_raw(x), src, dst))


def moveaxes(x, srcs, dsts):
    return _wrap(torch.movedim(_raw(x), list(srcs), list(dsts)))


def swapaxes(x, a: int, b: int):
    return _wrap(_raw(x).transpose(a, b))


def roll(x, shift, axis=None):
    return _wrap(torch.roll(_raw(x), shift, axis) if axis is not None else torch.roll(_raw(x).reshape(-1), shift).reshape(x.shape))


@dataclass
class ReduceSpec:
    op: str = "sum"        # sum | mean | min | max | prod | any | all
    keepdims: bool = False
    skipna: bool = False


def reduce_along_axis(x, axis: int, spec: ReduceSpec | None = None, mask=None):
    """``mask`` (same shape, non-zero = use) leaves the other elements out of the reduction, like missing values."""
    spec = spec or ReduceSpec()
    r = _raw(x)
    if mask is not None:
        import dataclasses
        r = torch.where(_raw(mask) != 0, r.double(), torch.full_like(r, float("nan"), dtype=torch.float64))
        spec = dataclasses.replace(spec, skipna=True) if dataclasses.is_dataclass(spec) else spec
    if spec.skipna and r.dtype.is_floating_point:
        fill = {"sum": 0.0, "mean": float("nan"), "min": float("inf"), "max": float("-inf"), "prod": 1.0}.get(spec.op, 0.0)
        if spec.op == "mean":
            return _wrap(torch.nanmean(r, dim=axis, keepdim=spec.keepdims))
        r = torch.where(torch.isnan(r), torch.full_like(r, fill), r)
    if spec.op == "sum":
        out = r.sum(axis, keepdim=spec.keepdims)
    elif spec.op == "mean":
        out = (r.double() if not r.dtype.is_floating_point else r).mean(axis, keepdim=spec.keepdims)
    elif spec.op == "min":
        out = r.min(axis, keepdim=spec.keepdims).values
    elif spec.op == "max":
        out = r.max(axis, keepdim=spec.keepdims).values
    elif spec.op == "prod":
        out = r.prod(axis, keepdim=spec.keepdims)
    elif spec.op == "any":
        out = (r != 0).any(axis, keepdim=spec.keepdims).to(torch.int64)
    elif spec.op == "all":
        out = (r != 0).all(axis, keepdim=spec.keepdims).to(torch.int64)
    else:
        raise ValueError(spec.op)
    return _wrap(out)


def cumsum(x, axis: int = -1):
    return _wrap(torch.cumsum(_raw(x), axis))


def cumprod(x, axis: int = -1):
    return _wrap(torch.cumprod(_raw(x), axis))


def quantile(x, q, axis=None, keepdims=False, axes=None, interpolation: str = "linear"):
    """``axes`` reduces over several axes at once (they are moved to the end and flattened); ``interpolation`` is
    linear / lower / higher / nearest / midpoint (legacy/src/momijo/tensor/axis.mojo:1098-1146)."""
    r = _raw(x).double()
    qq = torch.as_tensor(q, dtype=torch.float64)
    if axes:
        rank = r.dim()
        ax = sorted({a % rank for a in axes})
        keep = [d for d in range(rank) if d not in ax]
        flat = r.permute(keep + ax).reshape([r.shape[d] for d in keep] + [-1])
        out = torch.quantile(flat, qq, dim=-1, interpolation=interpolation)
        if keepdims:
            for a in ax:
                out = out.unsqueeze(a)
        return _wrap(out)
    if axis is None:
        return _wrap(torch.quantile(r, qq, interpolation=interpolation))
    return _wrap(torch.quantile(r, qq, dim=axis, keepdim=keepdims, interpolation=interpolation))


def percentile(x, p, axis=None, keepdims=False, axes=None, interpolation: str = "linear"):
    return quantile(x, torch.as_tensor(p, dtype=torch.float64) / 100.0, axis, keepdims, axes, interpolation)


def median(x, axis=None, keepdims=False, axes=None):
    return quantile(x, 0.5, axis, keepdims, axes)


def normalize(x, axis: int = -1, eps: float = 1e-12, axes=None):
    r = _raw(x).double()
    dims = tuple(axes) if axes else (list(range(r.dim())) if axis is None else axis)
    mu = r.mean(dims, keepdim=True)
    sd = r.std(dims, keepdim=True, unbiased=False)
    return _wrap((r - mu) / (sd + eps))


# ---- further reduction names of the reference (legacy/src/momijo/tensor/axis.mojo:53-1200) ------------------------
import math as _math  # noqa: E402


def isnan_f64(v: float) -> bool: return v != v                       # noqa: E704
def sqrt64(x: float) -> float: return _math.sqrt(x) if x > 0 else 0.0   # noqa: E704


def normalize_axes(axs, rank: int):
    """Negative axes wrapped, clamped into [0, rank - 1], duplicates removed, order kept."""
    out = []
    for a in axs:
        a = min(max(a + rank if a < 0 else a, 0), max(rank - 1, 0))
        if a not in out:
            out.append(a)
    return out


def shape_drop_axes(shape, axes):
    drop = set(normalize_axes(axes, len(shape)))
    return [d for i, d in enumerate(shape) if i not in drop]


drop_axes = shape_drop_axes


def axis_to_list(axis, axes_list, rank: int):
    """``axes_list`` wins over ``axis``; neither means all axes."""
    if axes_list is not None:
        return normalize_axes(list(axes_list), rank)
    if axis is not None:
        return normalize_axes([axis], rank)
    return list(range(rank))


_OPS = {0: "sum", 1: "mean", 2: "max", 3: "min", 4: "prod"}


def neutral(spec) -> float:
    op = getattr(spec, "op_id", None)
    return 1.0 if op == 4 or getattr(spec, "op", "") == "prod" else 0.0


def apply_acc(acc: float, v: float, spec, inited: bool):
    """One accumulation step of a reduction: (new accumulator, initialised flag). With skip-NaN mode a NaN
    sample leaves the state unchanged."""
    op = _OPS.get(getattr(spec, "op_id", None), getattr(spec, "op", "sum"))
    skip = getattr(spec, "nan_mode", 0) == 1 or getattr(spec, "skipna", False)
    if skip and v != v:
        return acc, inited
    if op in ("sum", "mean"):
        return acc + v, True
    if op == "prod":
        return acc * v, True
    if not inited:
        return v, True
    return (max(acc, v) if op == "max" else min(acc, v)), True


def _reduce(x, op: str, axis, keepdims, axes, skipna=False):
    r = _raw(x)
    dims = axis_to_list(axis, axes, r.dim())
    if skipna and r.dtype.is_floating_point:
        nan = torch.isnan(r)
        if op == "mean":
            cnt = (~nan).sum(dim=dims, keepdim=keepdims).clamp_min(1)
            return _wrap(torch.where(nan, torch.zeros_like(r), r).sum(dim=dims, keepdim=keepdims) / cnt)
        fill = {"sum": 0.0, "prod": 1.0, "max": float("-inf"), "min": float("inf")}[op]
        r = torch.where(nan, torch.full_like(r, fill), r)
    if op == "sum":
        return _wrap(r.sum(dim=dims, keepdim=keepdims))
    if op == "mean":
        return _wrap((r if r.dtype.is_floating_point else r.double()).mean(dim=dims, keepdim=keepdims))
    if op == "prod":
        out = r
        for d in sorted(dims, reverse=True):
            out = out.prod(dim=d, keepdim=keepdims)
        return _wrap(out)
    return _wrap(torch.amax(r, dim=dims, keepdim=keepdims) if op == "max" else torch.amin(r, dim=dims, keepdim=keepdims))


def reduce_sum(x, axis=None, keepdims=False, axes=None): return _reduce(x, "sum", axis, keepdims, axes)      # noqa: E704
def reduce_mean(x, axis=None, keepdims=False, axes=None): return _reduce(x, "mean", axis, keepdims, axes)    # noqa: E704
def reduce_max(x, axis=None, keepdims=False, axes=None): return _reduce(x, "max", axis, keepdims, axes)      # noqa: E704
def reduce_min(x, axis=None, keepdims=False, axes=None): return _reduce(x, "min", axis, keepdims, axes)      # noqa: E704
def reduce_prod(x, axis=None, keepdims=False, axes=None): return _reduce(x, "prod", axis, keepdims, axes)    # noqa: E704
def nan_sum(x, axis=None, keepdims=False, axes=None): return _reduce(x, "sum", axis, keepdims, axes, True)    # noqa: E704
def nan_mean(x, axis=None, keepdims=False, axes=None): return _reduce(x, "mean", axis, keepdims, axes, True)  # noqa: E704
def nan_max(x, axis=None, keepdims=False, axes=None): return _reduce(x, "max", axis, keepdims, axes, True)    # noqa: E704
def nan_min(x, axis=None, keepdims=False, axes=None): return _reduce(x, "min", axis, keepdims, axes, True)    # noqa: E704
def nan_prod(x, axis=None, keepdims=False, axes=None): return _reduce(x, "prod", axis, keepdims, axes, True)  # noqa: E704


def reduce_multi_axis(x, axes, keepdims: bool, spec, out=None):
    op = _OPS.get(getattr(spec, "op_id", None), getattr(spec, "op", "sum"))
    skip = getattr(spec, "nan_mode", 0) == 1 or getattr(spec, "skipna", False)
    return _reduce(x, op, None, keepdims, list(axes) if axes else None, skip)


def arg_reduce(x, axis=None, axes=None, mode: int = 1):
    """Index of the maximum (``mode`` 1) or minimum (``mode`` 0): over the flattened tensor when no axis is
    given, else along the (first) axis."""
    r = _raw(x)
    fn = torch.argmax if mode == 1 else torch.argmin
    if axis is None and axes is None:
        return _wrap(fn(r.reshape(-1)))
    return _wrap(fn(r, dim=axis_to_list(axis, axes, r.dim())[0]))


def _nanarg(x, axis, axes, largest: bool):
    r = _raw(x)
    if r.dtype.is_floating_point:
        r = torch.where(torch.isnan(r), torch.full_like(r, float("-inf") if largest else float("inf")), r)
    return arg_reduce(_wrap(r), axis, axes, 1 if largest else 0)


def nanargmax(x, axis=None, axes=None): return _nanarg(x, axis, axes, True)      # noqa: E704
def nanargmin(x, axis=None, axes=None): return _nanarg(x, axis, axes, False)     # noqa: E704


def minmax(x):
    """float64 tensor [min, max] over all elements ([0, 0] when empty)."""
    r = _raw(x).double().reshape(-1)
    return _wrap(torch.stack([r.min(), r.max()]) if r.numel() else torch.zeros(2, dtype=torch.float64))


def sum1d_contig(x) -> float:
    return float(_raw(x).double().sum())


def roll_one(x, ax: int, sft: int):
    r = _raw(x)
    return _wrap(r.clone() if r.dim() == 0 else torch.roll(r, sft, ax))


def roll_flat(x, shift: int):
    r = _raw(x)
    return _wrap(torch.roll(r.reshape(-1), shift).reshape(r.shape) if r.numel() else r.clone())


def roll_multi(x, shifts, axes):
    r = _raw(x)
    return _wrap(r.clone() if r.dim() == 0 else torch.roll(r, list(shifts), list(axes)))


def normalize_(x, axis=None, eps: float = 1e-12, axes=None) -> None:
    if axes:
        _raw(x).copy_(_raw(normalize(x, axis, eps, axes)).to(_raw(x).dtype))
        return
    from .math_compat import normalize_ as _n
    _n(x, axis, eps)


def partition(a: list, l: int, r: int, pivot: float):
    """Three-way partition of ``a[l..r]`` in place; returns (lt, gt) with a[l..lt-1] < pivot, a[lt..gt] == pivot,
    a[gt+1..r] > pivot."""
    i, lt, gt = l, l, r
    while i <= gt:
        if a[i] < pivot:
            a[lt], a[i] = a[i], a[lt]
            lt += 1
            i += 1
        elif a[i] > pivot:
            a[i], a[gt] = a[gt], a[i]
            gt -= 1
        else:
            i += 1
    return lt, gt


def select_kth(a: list, k: int) -> float:
    """k-th smallest (0-based) by quick-select; reorders ``a``."""
    l, r = 0, len(a) - 1
    while l <= r:
        lt, gt = partition(a, l, r, a[(l + r) // 2])
        if k < lt:
            r = lt - 1
        elif k > gt:
            l = gt + 1
        else:
            return a[k]
    return a[min(max(k, 0), len(a) - 1)] if a else 0.0


def quantile_1d_partial(xs, q: float, interpolation: str = "linear") -> float:
    """Quantile ``q`` in [0, 1] of a list via selection; ``interpolation`` is linear, lower, higher, nearest or
    midpoint. 0.0 for an empty list."""
    n = len(xs)
    if n == 0:
        return 0.0
    pos = min(max(q, 0.0), 1.0) * (n - 1)
    lo, hi = int(_math.floor(pos)), int(_math.ceil(pos))
    a = list(xs)
    vlo = select_kth(a, lo)
    vhi = select_kth(a, hi)
    if interpolation == "lower":
        return vlo
    if interpolation == "higher":
        return vhi
    if interpolation == "nearest":
        return vlo if pos - lo <= hi - pos else vhi
    if interpolation == "midpoint":
        return 0.5 * (vlo + vhi)
    return vlo + (vhi - vlo) * (pos - lo)


def unique(x, axis=None):
    """Distinct values in order of first appearance (flattened, as in the reference)."""
    r = _raw(x).reshape(-1)
    seen = list(dict.fromkeys(r.tolist()))
    return _wrap(torch.tensor(seen, dtype=r.dtype))


def bincount(x, minlength: int = 0):
    r = _raw(x).reshape(-1).long()
    r = r[r >= 0]
    return _wrap(torch.bincount(r, minlength=max(minlength, 0)))
