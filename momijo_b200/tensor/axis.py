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


def reduce_along_axis(x, axis: int, spec: ReduceSpec | None = None):
    spec = spec or ReduceSpec()
    r = _raw(x)
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


def quantile(x, q, axis=None, keepdims=False):
    r = _raw(x).double()
    qq = torch.as_tensor(q, dtype=torch.float64)
    return _wrap(torch.quantile(r, qq) if axis is None else torch.quantile(r, qq, dim=axis, keepdim=keepdims))


def percentile(x, p, axis=None, keepdims=False):
    return quantile(x, torch.as_tensor(p, dtype=torch.float64) / 100.0, axis, keepdims)


def median(x, axis=None, keepdims=False):
    return quantile(x, 0.5, axis, keepdims)


def normalize(x, axis: int = -1, eps: float = 1e-12):
    r = _raw(x).double()
    mu = r.mean(axis, keepdim=True)
    sd = r.std(axis, keepdim=True, unbiased=False)
    return _wrap((r - mu) / (sd + eps))
