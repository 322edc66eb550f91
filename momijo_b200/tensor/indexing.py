"""Indexing, gather/scatter/where/topk, triangular helpers, im2col and the tiled
``sgemm/dgemm`` names (legacy/src/momijo/tensor/indexing.mojo:279-3214)."""
from __future__ import annotations

import torch
import torch.nn.functional as tF

from .tensor import _mask, _raw, _wrap


def slice1d(x, start=0, stop=None, step=1):
    return _wrap(_raw(x)[start:stop:step])


def slice2d(x, r0=0, r1=None, c0=0, c1=None):
    return _wrap(_raw(x)[r0:r1, c0:c1])


def head(x, n=5):
    return _wrap(_raw(x)[:n])


def tail(x, n=5):
    return _wrap(_raw(x)[-n:] if n > 0 else _raw(x)[:0])


def slice_dim0(x, start, stop):
    return _wrap(_raw(x)[start:stop])


def plane(x, axis: int, index: int):
    return _wrap(_raw(x).select(axis, index))


def col(x, j: int):
    return _wrap(_raw(x)[:, j])


def row(x, i: int):
    return _wrap(_raw(x)[i])


def gather(x, axis: int, index):
    return _wrap(torch.gather(_raw(x), axis, _raw(index).long()))


def take(x, index):
    return _wrap(torch.take(_raw(x), _raw(index).long()))


def take_along_axis(x, index, axis: int):
    return _wrap(torch.take_along_dim(_raw(x), _raw(index).long(), axis))


def scatter(x, axis: int, index, src):
    return _wrap(_raw(x).scatter(axis, _raw(index).long(), _raw(src) if isinstance(src, torch.Tensor) else src))


def scatter_nd(shape, indices, updates):
    out = torch.zeros(list(shape), dtype=_raw(updates).dtype)
    idx = _raw(indices).long()
    out.index_put_(tuple(idx.t()), _raw(updates), accumulate=True)
    return _wrap(out)


def where(cond, a, b):
    """``cond`` may be an Int (0/1) or bool mask; same-shape fp32 CUDA tensors use the kernel."""
    c, ra = _raw(cond), _raw(a) if isinstance(a, torch.Tensor) else a
    rb = _raw(b) if isinstance(b, torch.Tensor) else b
    if (isinstance(ra, torch.Tensor) and isinstance(rb, torch.Tensor) and ra.is_cuda and ra.dtype == torch.float32
            and rb.dtype == torch.float32 and ra.shape == rb.shape == c.shape and ra.is_contiguous()
            and rb.is_contiguous()):
        from .. import _C

        ci = c.to(torch.int32).contiguous()
        out = torch.empty_like(ra)
        _C.call("mmj_where_f32", _C.ptr(ci), _C.ptr(ra), _C.ptr(rb), _C.ptr(out), ra.numel(), _C.current_stream())
        return _wrap(out)
    return _wrap(torch.where(_mask(c), ra, rb))


def nonzero(x):
    return _wrap(torch.nonzero(_raw(x)))


argwhere = nonzero


def tril(x, k: int = 0):
    return _wrap(torch.tril(_raw(x), k))


def triu(x, k: int = 0):
    return _wrap(torch.triu(_raw(x), k))


def diag(x, k: int = 0):
    return _wrap(torch.diag(_raw(x), k))


def topk(x, k: int, axis: int = -1, largest: bool = True):
    v, i = torch.topk(_raw(x), k, dim=axis, largest=largest)
    return _wrap(v), _wrap(i)


def im2col_core(x, kh, kw, sh=1, sw=1, ph=0, pw=0):
    cols = tF.unfold(_raw(x), (kh, kw), padding=(ph, pw), stride=(sh, sw))
    return _wrap(cols)


def col2im_core(cols, out_hw, kh, kw, sh=1, sw=1, ph=0, pw=0):
    return _wrap(tF.fold(_raw(cols), out_hw, (kh, kw), padding=(ph, pw), stride=(sh, sw)))


def select_tiles(m: int, n: int, k: int):
    """Tile sizes used by the GEMM kernel for an (m, n, k) problem."""
    from ..ops.gemm import pick_bn

    return 128, pick_bn(m, n), 64


def sgemm(a, b, alpha=1.0, beta=0.0, c=None):
    r = alpha * (_raw(a).float() @ _raw(b).float())
    return _wrap(r + beta * _raw(c).float() if c is not None else r)


def dgemm(a, b, alpha=1.0, beta=0.0, c=None):
    r = alpha * (_raw(a).double() @ _raw(b).double())
    return _wrap(r + beta * _raw(c).double() if c is not None else r)


def histogram(x, bins=10, lo=None, hi=None):
    r = _raw(x).double().reshape(-1)
    lo = float(r.min()) if lo is None else lo
    hi = float(r.max()) if hi is None else hi
    return _wrap(torch.histc(r, bins=bins, min=lo, max=hi).long()), _wrap(torch.linspace(lo, hi, bins + 1, dtype=torch.float64))


def infer_shape(nested) -> list:
    """Shape of a nested list (ragged input raises)."""
    shape, cur = [], nested
    while isinstance(cur, (list, tuple)):
        shape.append(len(cur))
        if not cur:
            break
        if any(isinstance(v, (list, tuple)) != isinstance(cur[0], (list, tuple)) or
               (isinstance(v, (list, tuple)) and len(v) != len(cur[0])) for v in cur):
            raise ValueError("ragged nested list")
        cur = cur[0]
    return shape
