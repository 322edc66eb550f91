"""``Tensor``: momijo's N-d array on top of ``torch.Tensor``.

The reference ``Tensor[T]`` is a strided array over a ``List[T]`` with ~230 methods
(legacy/src/momijo/tensor/tensor.mojo:776-6389). Here it is a ``torch.Tensor`` subclass, so every
torch operation (and autograd, and CUDA placement) works on it, plus the reference's method names
and its observable semantics:

* value semantics at API boundaries (``copy()``), views only from indexing / reshape / permute;
* promotion: Int (+,-,*) Int -> Int; anything with Float64 -> Float64; Float32 with Int ->
  Float32; true division and ``%`` of Int tensors give Float64; ``Int @ Int -> Float32``
  (tensor.mojo:3164-3167, 4311-4460);
* comparisons return Int (0/1) masks (used as ``Tensor[Int]`` in ``where``);
* string-spec selectors ``t[S("1:3, :")]`` (tensor.mojo:635-644).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .errors import ErrorKind, TensorError, compat

_INT = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool)


def _is_int(t) -> bool:
    return isinstance(t, torch.Tensor) and t.dtype in _INT


def _wrap(x):
    if isinstance(x, torch.Tensor) and not isinstance(x, Tensor):
        return x.as_subclass(Tensor)
    return x


def _raw(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, Tensor) else x


def _mask(m):
    """Accept Int (0/1) or bool masks."""
    m = _raw(m)
    return m if m.dtype == torch.bool else m != 0


class S:
    """String selector, e.g. ``t[S("1:3, :, -1")]`` or ``t[S("::2")]``."""

    def __init__(self, spec: str):
        self.spec = spec

    def to_index(self):
        out = []
        for part in self.spec.split(","):
            p = part.strip()
            if p == "...":
                out.append(Ellipsis)
            elif p in ("None", "newaxis"):
                out.append(None)
            elif ":" in p:
                f = [int(v) if v.strip() else None for v in p.split(":")]
                out.append(slice(*f))
            elif p.startswith("["):
                out.append([int(v) for v in p.strip("[]").split() if v] or [int(v) for v in p.strip("[]").split(";") if v])
            else:
                out.append(int(p))
        return tuple(out)


class _Shape(tuple):
    """Shape tuple that can also be called: the reference spells it ``x.shape()``."""

    def __call__(self):
        return list(self)

    def numel(self) -> int:
        n = 1
        for v in self:
            n *= v
        return n


class Tensor(torch.Tensor):
    # ---- construction -----------------------------------------------------------------------
    @staticmethod
    def __new__(cls, data=None, shape: Optional[Sequence[int]] = None, dtype=None, device=None):
        if data is None:
            t = torch.zeros(list(shape) if shape is not None else [0], dtype=dtype or torch.float32, device=device)
        elif isinstance(data, torch.Tensor):
            t = data.detach().clone() if dtype is None else data.detach().to(dtype)
        elif isinstance(data, (int, float, bool)) and shape is not None:
            t = torch.full(list(shape), data, dtype=dtype, device=device)
        else:
            t = torch.tensor(data, dtype=dtype, device=device)
            if t.dtype == torch.float64 and dtype is None and _all_py_float32(data):
                pass
        if shape is not None and not isinstance(data, (int, float, bool)) and data is not None:
            t = t.reshape(list(shape))
        return t.as_subclass(cls)

    def __init__(self, *a, **k):
        pass

    # ---- metadata ----------------------------------------------------------------------------
    @property
    def shape(self):
        return _Shape(torch.Tensor.shape.__get__(self))

    def transpose(self, *dims):
        """``transpose()`` swaps the last two axes (the reference's 2-D transpose); with arguments it is
        torch's ``transpose(dim0, dim1)``; more than two arguments permute."""
        if len(dims) == 0:
            return self if self.dim() < 2 else torch.Tensor.transpose(self, -2, -1)
        if len(dims) == 1 and isinstance(dims[0], (list, tuple)):
            return self.permute(*dims[0])
        if len(dims) > 2:
            return self.permute(*dims)
        return torch.Tensor.transpose(self, *dims)

    def numel_(self) -> int:
        return self.numel()

    def rank(self) -> int:
        return self.dim()

    def shape_list(self) -> List[int]:
        return list(self.shape)

    def strides(self) -> List[int]:
        return list(self.stride())

    def offset(self) -> int:
        return self.storage_offset()

    def is_contig(self) -> bool:
        return self.is_contiguous()

    def dtype_name(self) -> str:
        return str(self.dtype).replace("torch.", "")

    def copy(self):
        return self.clone()

    def share(self):
        return self.view(self.shape)

    def to_list(self):
        return self.tolist()

    def item_at(self, *idx):
        return self[tuple(idx)].item()

    # ---- indexing with string selectors ------------------------------------------------------
    def __getitem__(self, idx):
        if isinstance(idx, S):
            idx = idx.to_index()
        elif isinstance(idx, tuple):
            idx = tuple(j for i in idx for j in (i.to_index() if isinstance(i, S) else (i,)))
        src, idx = _resolve_negative_steps(self, idx)
        return torch.Tensor.__getitem__(src, idx)

    def __setitem__(self, idx, value):
        if isinstance(idx, S):
            idx = idx.to_index()
        elif isinstance(idx, tuple):
            idx = tuple(j for i in idx for j in (i.to_index() if isinstance(i, S) else (i,)))
        src, idx2, flips = _resolve_negative_steps(self, idx, want_flips=True)
        if flips:
            # negative-step selector: assign into the flipped copy (where the slice runs forwards) and
            # write the result back (the reference normalises such slices itself, tensor.mojo:676-718)
            torch.Tensor.__setitem__(src, idx2, value)
            with torch.no_grad():
                self.as_subclass(torch.Tensor).copy_(torch.flip(src.as_subclass(torch.Tensor), flips))
            return None
        return super().__setitem__(idx, value)

    # ---- promotion rules ------------------------------------------------------------------------
    def __truediv__(self, o):
        if _is_int(self) and (_is_int(o) or isinstance(o, (int, bool))):
            return _wrap(torch.true_divide(_raw(self).double(), _raw(o).double() if isinstance(o, torch.Tensor) else o))
        return super().__truediv__(o)

    def __rtruediv__(self, o):
        if _is_int(self) and isinstance(o, (int, bool)):
            return _wrap(o / _raw(self).double())
        return super().__rtruediv__(o)

    def __mod__(self, o):
        if _is_int(self) and (_is_int(o) or isinstance(o, (int, bool))):
            return _wrap(torch.remainder(_raw(self).double(), _raw(o).double() if isinstance(o, torch.Tensor) else o))
        return super().__mod__(o)

    def __matmul__(self, o):
        if _is_int(self) and _is_int(o):
            return _wrap(_raw(self).float() @ _raw(o).float())
        return super().__matmul__(o)

    def _cmp(self, o, fn):
        return _wrap(fn(_raw(self), _raw(o)).to(torch.int64))

    def __eq__(self, o):
        return self._cmp(o, torch.eq) if isinstance(o, (torch.Tensor, int, float, bool)) else NotImplemented

    def __ne__(self, o):
        return self._cmp(o, torch.ne) if isinstance(o, (torch.Tensor, int, float, bool)) else NotImplemented

    def __lt__(self, o):
        return self._cmp(o, torch.lt)

    def __le__(self, o):
        return self._cmp(o, torch.le)

    def __gt__(self, o):
        return self._cmp(o, torch.gt)

    def __ge__(self, o):
        return self._cmp(o, torch.ge)

    __hash__ = torch.Tensor.__hash__

    # ---- scalar arithmetic names ------------------------------------------------------------------
    def add_scalar(self, s):
        return self + s

    def sub_scalar(self, s):
        return self - s

    def mul_scalar(self, s):
        return self * s

    def div_scalar(self, s):
        return self / s

    def pow_scalar(self, s):
        return self ** s

    def rsub_scalar(self, s):
        return s - self

    def rdiv_scalar(self, s):
        return s / self

    def eq_scalar(self, s):
        return self == s

    def ne_scalar(self, s):
        return self != s

    def lt_scalar(self, s):
        return self < s

    def le_scalar(self, s):
        return self <= s

    def gt_scalar(self, s):
        return self > s

    def ge_scalar(self, s):
        return self >= s

    def maximum_scalar(self, s):
        return _wrap(torch.clamp(_raw(self), min=s))

    def minimum_scalar(self, s):
        return _wrap(torch.clamp(_raw(self), max=s))

    # ---- logical / bitwise (Int masks) ------------------------------------------------------------
    def logical_and_(self, o):
        return _wrap((_mask(self) & _mask(o)).to(torch.int64))

    def logical_or_(self, o):
        return _wrap((_mask(self) | _mask(o)).to(torch.int64))

    def logical_xor_(self, o):
        return _wrap((_mask(self) ^ _mask(o)).to(torch.int64))

    def logical_not_(self):
        return _wrap((~_mask(self)).to(torch.int64))

    and_t = logical_and_
    or_t = logical_or_
    xor_t = logical_xor_
    not_t = logical_not_

    # ---- unary math (names missing from torch) ---------------------------------------------------
    def gelu(self):
        return _wrap(torch.nn.functional.gelu(_raw(self), approximate="tanh"))

    def silu(self):
        return _wrap(torch.nn.functional.silu(_raw(self)))

    def elu(self, alpha=1.0):
        return _wrap(torch.nn.functional.elu(_raw(self), alpha))

    def selu(self):
        return _wrap(torch.nn.functional.selu(_raw(self)))

    def leaky_relu(self, slope=0.01):
        return _wrap(torch.nn.functional.leaky_relu(_raw(self), slope))

    # ---- reductions ----------------------------------------------------------------------------------
    def sum_all(self):
        return self.sum().item()

    def mean_all(self):
        return _raw(self).double().mean().item() if self.numel() else 0.0

    def std_all(self, unbiased: bool = False):
        return _raw(self).double().std(unbiased=unbiased).item() if self.numel() else 0.0

    def var_all(self, unbiased: bool = False):
        return _raw(self).double().var(unbiased=unbiased).item() if self.numel() else 0.0

    def min_all(self):
        return self.min().item()

    def max_all(self):
        return self.max().item()

    def prod_all(self):
        return self.prod().item()

    def any_(self):
        return bool(_mask(self).any())

    def all_(self):
        return bool(_mask(self).all())

    def nansum(self, axis=None, keepdims=False):
        return _wrap(torch.nansum(_raw(self)) if axis is None else torch.nansum(_raw(self), dim=axis, keepdim=keepdims))

    def nanmean(self, axis=None, keepdims=False):
        return _wrap(torch.nanmean(_raw(self)) if axis is None else torch.nanmean(_raw(self), dim=axis, keepdim=keepdims))

    def nanmin(self, axis=None):
        """True nan-aware minimum (the reference's method calls ``nansum`` by mistake,
        tensor.mojo:3239-3261)."""
        r = _raw(self)
        if r.dtype.is_floating_point:
            r = torch.where(torch.isnan(r), torch.full_like(r, float("inf")), r)
        return _wrap(r.min() if axis is None else r.min(dim=axis).values)

    def nanmax(self, axis=None):
        r = _raw(self)
        if r.dtype.is_floating_point:
            r = torch.where(torch.isnan(r), torch.full_like(r, float("-inf")), r)
        return _wrap(r.max() if axis is None else r.max(dim=axis).values)

    # ---- linear algebra -----------------------------------------------------------------------------
    def matmul_vec(self, v):
        return self @ v

    def tensordot(self, o, axes: int = 1):
        return _wrap(torch.tensordot(_raw(self), _raw(o), dims=axes))

    def solve(self, b):
        return _wrap(torch.linalg.solve(_raw(self), _raw(b)))

    def inv(self):
        return _wrap(torch.linalg.inv(_raw(self)))

    def qr(self):
        q, r = torch.linalg.qr(_raw(self))
        return _wrap(q), _wrap(r)

    def svd(self):
        u, s, vh = torch.linalg.svd(_raw(self), full_matrices=False)
        return _wrap(u), _wrap(s), _wrap(vh)

    def cholesky(self):
        return _wrap(torch.linalg.cholesky(_raw(self)))

    def det(self):
        return torch.linalg.det(_raw(self)).item()

    # ---- sorting / sets / counting ---------------------------------------------------------------------
    def sort_(self, axis: int = -1, descending: bool = False):
        return _wrap(torch.sort(_raw(self), dim=axis, descending=descending).values)

    def argsort_(self, axis: int = -1, descending: bool = False):
        return _wrap(torch.argsort(_raw(self), dim=axis, descending=descending))

    def unique_(self):
        return _wrap(torch.unique(_raw(self)))

    def topk_(self, k: int, axis: int = -1, largest: bool = True):
        v, i = torch.topk(_raw(self), k, dim=axis, largest=largest)
        return _wrap(v), _wrap(i)

    def bincount_(self, minlength: int = 0):
        return _wrap(torch.bincount(_raw(self).long().reshape(-1), minlength=minlength))

    def histogram_(self, bins: int = 10, lo=None, hi=None):
        x = _raw(self).double().reshape(-1)
        lo = float(x.min()) if lo is None else lo
        hi = float(x.max()) if hi is None else hi
        h = torch.histc(x, bins=bins, min=lo, max=hi)
        edges = torch.linspace(lo, hi, bins + 1, dtype=torch.float64)
        return _wrap(h.long()), _wrap(edges)

    def digitize(self, bins, right: bool = False):
        return _wrap(torch.bucketize(_raw(self), _raw(bins), right=not right if False else right))

    def union(self, o):
        return _wrap(torch.unique(torch.cat([_raw(self).reshape(-1), _raw(o).reshape(-1)])))

    def intersect(self, o):
        a, b = torch.unique(_raw(self)), torch.unique(_raw(o))
        return _wrap(a[torch.isin(a, b)])

    def setdiff(self, o):
        a = torch.unique(_raw(self))
        return _wrap(a[~torch.isin(a, _raw(o))])

    def setxor(self, o):
        a, b = torch.unique(_raw(self)), torch.unique(_raw(o))
        return _wrap(torch.unique(torch.cat([a[~torch.isin(a, b)], b[~torch.isin(b, a)]])))

    def isin_(self, o):
        return _wrap(torch.isin(_raw(self), _raw(o)).to(torch.int64))

    # ---- selection / scatter ------------------------------------------------------------------------------
    def masked_select_(self, m):
        return _wrap(torch.masked_select(_raw(self), _mask(m)))

    def masked_fill_value(self, m, v):
        return _wrap(_raw(self).masked_fill(_mask(m), v))

    boolean_select = masked_select_

    def take_(self, idx):
        return _wrap(torch.take(_raw(self), _raw(idx).long()))

    def put(self, idx, values):
        out = _raw(self).clone()
        out.reshape(-1)[_raw(idx).long()] = _raw(values).to(out.dtype)
        return _wrap(out)

    def gather_(self, axis: int, idx):
        return _wrap(torch.gather(_raw(self), axis, _raw(idx).long()))

    def scatter_value(self, axis: int, idx, src):
        return _wrap(_raw(self).scatter(axis, _raw(idx).long(), _raw(src) if isinstance(src, torch.Tensor) else src))

    def scatter_add_value(self, axis: int, idx, src):
        return _wrap(_raw(self).scatter_add(axis, _raw(idx).long(), _raw(src)))

    def one_hot(self, num_classes: int, dtype=torch.float32):
        idx = _raw(self).long()
        if idx.is_cuda and dtype == torch.float32 and idx.dim() == 1:
            from .. import _C

            out = torch.empty((idx.numel(), num_classes), dtype=torch.float32, device=idx.device)
            _C.call("mmj_one_hot_f32", _C.ptr(idx.contiguous()), _C.ptr(out), idx.numel(), num_classes,
                    _C.current_stream())
            return _wrap(out)
        return _wrap(torch.nn.functional.one_hot(idx, num_classes).to(dtype))

    def clip(self, lo=None, hi=None):
        return _wrap(torch.clamp(_raw(self), lo, hi))

    clamped = clip

    # ---- RNG fills (explicit seeds) ---------------------------------------------------------------------------
    def uniform_seeded(self, lo=0.0, hi=1.0, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        v = torch.empty(self.shape, dtype=torch.float64).uniform_(lo, hi, generator=g)
        with torch.no_grad():
            self.copy_(v.to(self.dtype))
        return self

    def bernoulli_seeded(self, p=0.5, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        return _wrap((torch.rand(self.shape, generator=g) < p).to(torch.int64))

    def multinomial_seeded(self, n: int, replacement: bool = True, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        return _wrap(torch.multinomial(_raw(self).float().cpu(), n, replacement, generator=g))

    # ---- shape ops with reference names ------------------------------------------------------------------------
    def reshape_infer(self, shape):
        return self.reshape(list(shape))

    def transpose2d(self):
        if self.dim() != 2:
            raise TensorError(ErrorKind.SHAPE, "transpose2d needs a 2-D tensor")
        x = _raw(self)
        if x.is_cuda and x.is_contiguous() and x.element_size() in (2, 4):
            from .. import _C

            out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
            _C.call("mmj_transpose2d", _C.ptr(x), _C.ptr(out), x.shape[0], x.shape[1], x.element_size(),
                    _C.current_stream())
            return _wrap(out)
        return _wrap(x.t().contiguous())

    def flatten_all(self):
        return self.reshape(-1)

    def astype(self, dtype):
        from .cast import astype

        return astype(self, dtype)

    def __repr__(self, *a, **k):
        from .printing import tensor_to_string

        return tensor_to_string(self)


def _all_py_float32(data) -> bool:
    return False


def _resolve_negative_steps(t, idx, want_flips=False):
    """torch has no negative-step slices: flip the affected axes and rewrite the slice so that the
    result equals NumPy's (the reference normalises such slices itself, tensor.mojo:676-718)."""
    keys = idx if isinstance(idx, tuple) else (idx,)
    if not any(isinstance(k, slice) and k.step is not None and k.step < 0 for k in keys):
        return (t, idx, []) if want_flips else (t, idx)
    n_real = sum(1 for k in keys if k is not None and k is not Ellipsis)
    out, dim, flips = [], 0, []
    for k in keys:
        if k is None:
            out.append(k)
            continue
        if k is Ellipsis:
            dim += t.dim() - n_real
            out.append(k)
            continue
        if isinstance(k, slice) and k.step is not None and k.step < 0:
            n = t.shape[dim]
            start, stop, step = k.indices(n)
            flips.append(dim)
            out.append(slice(n - 1 - start, n - 1 - stop, -step))
        else:
            out.append(k)
        dim += 1
    src = torch.flip(t.as_subclass(torch.Tensor), flips).as_subclass(type(t))
    new_idx = tuple(out) if isinstance(idx, tuple) else out[0]
    return (src, new_idx, flips) if want_flips else (src, new_idx)


def as_tensor(x) -> Tensor:
    if isinstance(x, Tensor):
        return x
    if isinstance(x, torch.Tensor):
        return x.as_subclass(Tensor)
    return Tensor(x)


# Code written against the reference often does ``from momijo.tensor import tensor`` and then calls
# ``tensor.randn([4, 10])``, ``tensor.matmul(a, b)``, ``tensor.maximum_scalar(x, 0.0)``
# (legacy/src/momijo/learn/examples/learn/*.mojo). Names that are not defined in this module are looked
# up in the package (creation, math, transform, ... re-exports) and then as ``Tensor`` methods.
def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    import importlib

    pkg = importlib.import_module(__package__)
    if name in pkg.__dict__:
        return pkg.__dict__[name]
    if hasattr(Tensor, name):
        meth = getattr(Tensor, name)

        def free(x, *a, **kw):
            return meth(as_tensor(x), *a, **kw)
        free.__name__ = name
        return free
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


# ---- selector records and storage sharing (legacy/src/momijo/tensor/tensor.mojo:635-790) -----------------------------
class StrIndex:
    """A textual index such as ``"1:3, ::2"``; ``S(spec)`` turns the same text into slice keys."""

    def __init__(self, spec: str):
        self.spec = spec

    def keys(self):
        return S(self.spec)


class EllipsisSpec:
    """Stands for ``...`` in a list of selectors."""


def make_fancy_sel(js):
    from .helpers import IndexSel
    return IndexSel(fancy=list(js))


def clone_sel(x):
    """Independent copy of a selector (its index list is copied, not aliased)."""
    from .helpers import IndexSel, SliceSpec
    sl = SliceSpec(x.slice.start, x.slice.stop, x.slice.step) if x.slice is not None else None
    return IndexSel(x.index, sl, list(x.fancy) if x.fancy is not None else None)


def share(data, shape, strides, offset: int = 0):
    """Tensor over existing storage (a torch tensor, or a list that is copied once) with explicit shape, element
    strides and offset; no element is copied when ``data`` is a tensor."""
    base = _raw(data) if isinstance(data, (torch.Tensor, Tensor)) else torch.tensor(list(data))
    return _wrap(torch.as_strided(base.reshape(-1), list(shape), list(strides), offset))
