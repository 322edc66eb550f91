"""Indexing, gather/scatter/where/topk, triangular helpers, im2col and the tiled
``sgemm/dgemm`` names (legacy/src/momijo/tensor/indexing.mojo:279-3214)."""
from __future__ import annotations

import torch
import torch.nn.functional as tF

from .tensor import _mask, _raw, _wrap


def slice1d(x, start=0, stop=None, step=1):
    return _wrap(_raw(x)[start:stop:step])


def slice2d(x, r0=0, r1=None, c0=0, c1=None, rs: int = 1, cs: int = 1):
    return _wrap(_raw(x)[r0:r1:rs, c0:c1:cs])


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


def take(x, index, axis: int = None):
    """Flat take, or rows / columns along ``axis`` (legacy/src/momijo/tensor/indexing.mojo:1571-1573)."""
    idx = (_raw(index) if isinstance(index, torch.Tensor) else torch.as_tensor(index)).long()
    if axis is None:
        return _wrap(torch.take(_raw(x), idx))
    return _wrap(torch.index_select(_raw(x), axis, idx.reshape(-1)))


def take_along_axis(x, index, axis: int):
    return _wrap(torch.take_along_dim(_raw(x), _raw(index).long(), axis))


def scatter(x, axis: int, index, src):
    return _wrap(_raw(x).scatter(axis, _raw(index).long(), _raw(src) if isinstance(src, torch.Tensor) else src))


def scatter_nd(shape, indices, updates):
    out = torch.zeros(list(shape), dtype=_raw(updates).dtype)
    idx = _raw(indices).long()
    out.index_put_(tuple(idx.t()), _raw(updates), accumulate=True)
    return _wrap(out)


def where(cond, a, b, from_f64=None):
    """``cond`` may be an Int (0/1) or bool mask; same-shape fp32 CUDA tensors use the kernel. ``from_f64`` (the
    reference's element converter) is accepted and not needed: dtypes follow the operands."""
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


def select_tiles(m: int, n: int, k: int, is_f64: bool = False):
    """Tile sizes used by the GEMM kernel for an (m, n, k) problem (``is_f64`` does not change them here)."""
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


# ---- further indexing names of the reference (legacy/src/momijo/tensor/indexing.mojo:279-2800) --------------------
def tensor_slice(x, begin, end, step=None):
    """Copy of ``x[begin[i]:end[i]:step[i]]`` over the leading axes (missing steps are 1)."""
    step = step or [1] * len(begin)
    key = tuple(slice(b, e, s or 1) for b, e, s in zip(begin, end, step))
    return _wrap(_raw(x)[key].clone())


def slice_view(x, begin, end, step=None):
    """Same selection as a view sharing storage with ``x``."""
    step = step or [1] * len(begin)
    return _wrap(_raw(x)[tuple(slice(b, e, s or 1) for b, e, s in zip(begin, end, step))])


def slice3d(t, d: int, r0: int = 0, r1: int = 0, c0: int = 0, c1: int = 0, rs: int = 1, cs: int = 1):
    """Rows r0:r1 and columns c0:c1 of plane ``d`` of a [D, R, C] tensor (an end of 0 means "to the end")."""
    raw = _raw(t)
    return _wrap(raw[d, r0:(r1 or raw.shape[1]):rs, c0:(c1 or raw.shape[2]):cs].clone())


def slice4d(t, a0, a1, b0, b1, c0, c1, d0, d1, as_=1, bs_=1, cs_=1, ds_=1):
    return _wrap(_raw(t)[a0:a1:as_, b0:b1:bs_, c0:c1:cs_, d0:d1:ds_].clone())


def get_last_dim_plane3(a, dim: int, index: int):
    """``a[:, :, index]`` of a rank-3 tensor (``dim`` must be 2); an empty [0, 0] tensor otherwise."""
    raw = _raw(a)
    if raw.dim() != 3 or dim != 2:
        return _wrap(torch.zeros(0, 0, dtype=raw.dtype))
    return _wrap(raw[:, :, index].clone())


def assign_last_dim_plane3(a, dim: int, index: int, rhs):
    raw = _raw(a)
    if raw.dim() == 3 and dim == 2:
        raw[:, :, index] = _raw(rhs)
    return a


def get_last_dim_plane4(a, dim: int, index: int):
    raw = _raw(a)
    if raw.dim() != 4 or dim != 3:
        return _wrap(torch.zeros(0, 0, 0, dtype=raw.dtype))
    return _wrap(raw[..., index].clone())


def assign_last_dim_plane4(a, dim: int, index: int, rhs):
    raw = _raw(a)
    if raw.dim() == 4 and dim == 3:
        raw[..., index] = _raw(rhs)
    return a


def getitem(x, idx: int):
    """Element ``idx`` in row-major order, as a Python scalar."""
    return _raw(x).reshape(-1)[idx].item()


def setitem(x, idx: int, v) -> None:
    """Set element ``idx`` (row-major order) in place."""
    raw = _raw(x)
    if raw.is_contiguous():
        raw.view(-1)[idx] = v
    else:
        flat = raw.reshape(-1).clone()
        flat[idx] = v
        raw.copy_(flat.reshape(raw.shape))


def item(x):
    """The first element as a Python scalar (0 for an empty tensor)."""
    raw = _raw(x)
    return raw.reshape(-1)[0].item() if raw.numel() else (False if raw.dtype == torch.bool else 0)


def at(x, i: int, j: int):
    raw = _raw(x)
    return raw.reshape(-1)[0].item() if raw.dim() < 2 else raw[i, j].item()


def set_at(x, i: int, j: int, v) -> None:
    raw = _raw(x)
    if raw.dim() < 2:
        raw.reshape(-1)[0] = v
    else:
        raw[i, j] = v


def fill(x, v) -> None:
    _raw(x).fill_(v)


def diagflat(x):
    return _wrap(torch.diagflat(_raw(x).reshape(-1)))


def fill_diagonal(x, v, k: int = 0) -> None:
    """Set the k-th diagonal of the last two axes in place (rank below 2: nothing happens)."""
    raw = _raw(x)
    if raw.dim() >= 2:
        torch.diagonal(raw, offset=k, dim1=-2, dim2=-1).fill_(v)


def band(x, k1: int, k2: int):
    """Keep the diagonals -k1 .. +k2 of the last two axes, zero elsewhere (negative bounds mean unbounded)."""
    raw = _raw(x)
    if raw.dim() < 2:
        return _wrap(raw.clone())
    out = raw.clone()
    if k1 >= 0:
        out = torch.triu(out, -k1)
    if k2 >= 0:
        out = torch.tril(out, k2)
    return _wrap(out)


def masked_select(x, mask):
    """1-D tensor of the elements where the (broadcast) mask is non-zero."""
    raw, m = torch.broadcast_tensors(_raw(x), _raw(mask) != 0)
    return _wrap(raw[m])


def masked_fill(x, mask, value) -> None:
    raw = _raw(x)
    raw.masked_fill_((_raw(mask) != 0).expand_as(raw), value)


def put(x, indices, values) -> None:
    """Write ``values`` at the row-major positions ``indices`` in place."""
    raw = _raw(x)
    idx = torch.as_tensor(_raw(indices) if hasattr(indices, "shape") else list(indices), dtype=torch.long)
    vals = _raw(values) if hasattr(values, "shape") else torch.as_tensor(values)
    flat = raw.reshape(-1).clone()
    flat[idx] = vals.to(raw.dtype).reshape(-1) if vals.dim() else vals.to(raw.dtype)
    raw.copy_(flat.reshape(raw.shape))


def take1d(t, indices):
    """Rows ``indices`` along the first axis."""
    return _wrap(_raw(t)[torch.as_tensor(list(indices), dtype=torch.long)])


def argwhere_any(x):
    """int32 [n, rank] coordinates of the non-zero elements of any tensor-like."""
    raw = _raw(getattr(x, "tensor", x)) if not isinstance(x, torch.Tensor) else x
    return _wrap(torch.nonzero(raw).to(torch.int32))


def tensor_from_flat(data, shape):
    return _wrap(torch.tensor(list(data)).reshape(list(shape)))


def where_f32(cond, x, y):
    return where(cond, x, y)


where_f32_auto = where_f32_cpu = where_f32_gpu = where_f64 = where_int = where_f32


def is_2d_f32(x) -> bool: return _raw(x).dim() == 2         # noqa: E704
def rows_f32(x) -> int: return int(_raw(x).shape[0])        # noqa: E704
def cols_f32(x) -> int: return int(_raw(x).shape[1])        # noqa: E704


is_2d_f64, rows_f64, cols_f64 = is_2d_f32, rows_f32, cols_f32


def check_sgemm_contract(a, b, c) -> bool:
    """a [m, k], b [k, n], c [m, n]."""
    if not (is_2d_f32(a) and is_2d_f32(b) and is_2d_f32(c)):
        return False
    return cols_f32(a) == rows_f32(b) and rows_f32(c) == rows_f32(a) and cols_f32(c) == cols_f32(b)


check_dgemm_contract = check_sgemm_contract


def zero_out_f32(c) -> None:
    _raw(c).zero_()


def scale_inplace_f32(c, beta: float) -> None:
    if beta == 0.0:
        _raw(c).zero_()
    elif beta != 1.0:
        _raw(c).mul_(beta)


zero_out_f64, scale_inplace_f64 = zero_out_f32, scale_inplace_f32


def sgemm_contig_kernel_base(A, B, C, alpha: float, beta: float, baseA: int = 0, baseB: int = 0, baseC: int = 0) -> bool:
    """C <- alpha * A @ B + beta * C in place; False when the shapes do not fit. The base offsets of the
    reference's flat-buffer kernel must be 0 here (tensors carry their own offsets)."""
    if not check_sgemm_contract(A, B, C) or baseA or baseB or baseC:
        return False
    c = _raw(C)
    c.copy_(alpha * (_raw(A).to(c.dtype) @ _raw(B).to(c.dtype)) + (beta * c if beta != 0.0 else 0.0))
    return True


sgemm_strided_kernel_base = dgemm_contig_kernel_base = dgemm_strided_kernel_base = sgemm_contig_kernel_base


def ravel_index_with_offset(idx, strides, offset: int) -> int:
    return offset + sum(int(i) * int(s) for i, s in zip(idx, strides))


def lin_index(idx, strides) -> int:
    return ravel_index_with_offset(idx, strides, 0)


def norm_range(start: int, stop: int, step: int, dim: int):
    """Positions selected by ``start:stop:step`` on an axis of length ``dim`` (a zero step counts as 1)."""
    return list(range(*slice(start, stop, step or 1).indices(dim)))


def list_select_one(xs, index: int):
    """One-element list with ``xs[index]`` (negative indices from the end, clamped); [] for an empty list."""
    n = len(xs)
    if n == 0:
        return []
    i = index + n if index < 0 else index
    return [xs[min(max(i, 0), n - 1)]]


def list_slice_generic(xs, start: int, stop: int, step: int = 1):
    return list(xs[slice(start, stop, step or 1)])


# The extents the reference passes after the nested list (n0, n1, ...) are implied by the list itself here.
def flatten_2d(xs, *dims): return [v for r in xs for v in r]                                   # noqa: E704
def flatten_3d(xs, *dims): return [v for a in xs for r in a for v in r]                        # noqa: E704
def flatten_4d(xs, *dims): return [v for a in xs for b in a for r in b for v in r]             # noqa: E704
def flatten_5d(xs, *dims): return [v for a in xs for b in a for c in b for r in c for v in r]  # noqa: E704
def infer_shape_1d(xs): return [len(xs)]                                                # noqa: E704
def infer_shape_2d(xs): return [len(xs), len(xs[0]) if xs else 0]                       # noqa: E704
def infer_shape_3d(xs): return infer_shape_2d(xs) + [len(xs[0][0]) if xs and xs[0] else 0]          # noqa: E704
def infer_shape_4d(xs): return infer_shape_3d(xs) + [len(xs[0][0][0]) if xs and xs[0] and xs[0][0] else 0]   # noqa: E704
def infer_shape_5d(xs): return infer_shape_4d(xs) + [len(xs[0][0][0][0])]               # noqa: E704


def histogram_core(values, bins: int, lo: float, hi: float):
    """Counts over ``bins`` equal-width bins of [lo, hi] (the right edge belongs to the last bin)."""
    counts = [0] * max(bins, 0)
    if bins <= 0 or hi <= lo:
        return counts
    w = (hi - lo) / bins
    for v in values:
        if lo <= v <= hi:
            counts[min(int((v - lo) / w), bins - 1)] += 1
    return counts


def histogram2d_core(xs, ys, bins_x: int, bins_y: int, x_lo, x_hi, y_lo, y_hi):
    out = [[0] * max(bins_y, 0) for _ in range(max(bins_x, 0))]
    if bins_x <= 0 or bins_y <= 0 or x_hi <= x_lo or y_hi <= y_lo:
        return out
    wx, wy = (x_hi - x_lo) / bins_x, (y_hi - y_lo) / bins_y
    for x, y in zip(xs, ys):
        if x_lo <= x <= x_hi and y_lo <= y <= y_hi:
            out[min(int((x - x_lo) / wx), bins_x - 1)][min(int((y - y_lo) / wy), bins_y - 1)] += 1
    return out


class Shape(list):
    """List of extents with ``numel`` and ``rank``."""

    def numel(self) -> int:
        n = 1
        for d in self:
            n *= d
        return n

    def rank(self) -> int:
        return len(self)

    ndim = rank

    @property
    def dims(self):
        return list(self)


class NDIter:
    """Row-major walk over the coordinates of a shape. Works as a Python iterable and through the reference's cursor
    calls ``next`` / ``next_inplace`` / ``reset`` (legacy/src/momijo/tensor/indexing.mojo:123-196); a rank-0 shape
    yields one empty coordinate."""

    def __init__(self, shape):
        self.shape = Shape(shape)
        self.reset()

    def reset(self) -> None:
        self.idx = [0] * len(self.shape)
        self.started = False
        self.finished = any(d <= 0 for d in self.shape)

    def next_inplace(self, out_idx: list) -> bool:
        if self.finished:
            return False
        if not self.started:
            self.started = True
            if len(self.shape) == 0:
                self.finished = True
            out_idx[:] = self.idx
            return True
        for ax in range(len(self.shape) - 1, -1, -1):
            self.idx[ax] += 1
            if self.idx[ax] < self.shape[ax]:
                out_idx[:] = self.idx
                return True
            self.idx[ax] = 0
        self.finished = True
        return False

    def next(self):
        out: list = []
        ok = self.next_inplace(out)
        return ok, out

    def __iter__(self):
        it = NDIter(self.shape)
        while True:
            ok, c = it.next()
            if not ok:
                return
            yield c


class NDLinearIter:
    """The same walk, also giving the linear offset of each coordinate in a strided layout
    (indexing.mojo:198-270). Iterating yields the offsets."""

    def __init__(self, shape, strides=None, offset: int = 0):
        if strides is None or isinstance(strides, LayoutView):
            view = strides
            self.strides = list(view.strides) if view is not None else []
            offset = view.offset if view is not None else 0
        else:
            self.strides = list(strides)
        self.shape, self.offset = Shape(shape), offset
        self._it = NDIter(self.shape)

    def reset(self) -> None:
        self._it.reset()

    def next_inplace(self, out_idx: list):
        ok = self._it.next_inplace(out_idx)
        return ok, (ravel_index_with_offset(out_idx, self.strides, self.offset) if ok else 0)

    def next(self):
        out: list = []
        ok, lin = self.next_inplace(out)
        return ok, out, lin

    def __iter__(self):
        return (ravel_index_with_offset(c, self.strides, self.offset) for c in NDIter(self.shape))


class LayoutView:
    """Shape, strides and offset of a tensor without its data."""

    def __init__(self, x):
        raw = _raw(x)
        self.shape, self.strides, self.offset = list(raw.shape), list(raw.stride()), raw.storage_offset()

    def is_contiguous(self) -> bool:
        exp, acc = [], 1
        for d in reversed(self.shape):
            exp.append(acc)
            acc *= d
        return list(reversed(exp)) == self.strides
