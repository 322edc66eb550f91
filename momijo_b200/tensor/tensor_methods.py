"""Method forms of the free functions on ``Tensor`` (legacy/src/momijo/tensor/tensor.mojo:783-6350): selector
builders, selector-based reads and writes, storage builders (append then ``set_shape_row_major``), bitwise /
shift / modulo spellings, dtype conversions and set operations. Each is a thin binding to the free function
that already implements it; attaching them here keeps the class body in ``tensor.py`` readable."""
from __future__ import annotations

from typing import List, Sequence

import torch

from . import helpers as H
from .tensor import Tensor, _raw, _wrap


def _key(sels):
    return tuple(s.to_key() if hasattr(s, "to_key") else (s.to_slice() if hasattr(s, "to_slice") else s) for s in sels)


# ---- selector builders (tensor.mojo:918-926, 2645-2660, 6337-6348) -----------------------------------------
def idx(self, i: int):
    return H.make_index_sel(i)


def slc(self, a: int, b: int, step: int = 1):
    return H.make_slice_sel((a, b, step))


def all_axis(self):
    return H.IndexSel(slice=H.SliceSpec())


def rng(self, a: int, b: int, step: int = 1):
    return H.make_slice_sel((a, b, step))


def reange(self, a: int, b: int):
    return H.make_slice_sel((a, b, 1))


def full(self, axis: int):
    n = self.dim()
    return H.SliceSpec(0, int(self.size(axis % n if n else 0)), 1)


def pad_full_axes(self, sels):
    d = self.dim()
    out = [H.clone_sel(s) if hasattr(H, "clone_sel") else s for s in list(sels)[:d]]
    while len(out) < d:
        out.append(all_axis(self))
    return out


# ---- selector reads / writes (tensor.mojo:986-1019, 1875-2004, 2699-2896) ----------------------------------
def select_view(self, sels):
    return _wrap(_raw(self)[_key(pad_full_axes(self, sels))])


def select(self, sels):
    return select_view(self, sels)


def select_copy(self, sels):
    return _wrap(_raw(self)[_key(pad_full_axes(self, sels))].clone())


def select_set_scalar(self, sels, value) -> None:
    _raw(self)[_key(pad_full_axes(self, sels))] = value


def select_set_tensor(self, sels, src) -> None:
    _raw(self)[_key(pad_full_axes(self, sels))] = _raw(src).to(self.dtype)


def slice_(self, specs):
    """A dense copy of the box named by one (start, stop, step) per axis (tensor.mojo:2699-2800)."""
    key = tuple(slice(*s) if isinstance(s, (tuple, list)) else s.to_slice() for s in specs)
    return _wrap(_raw(self)[key].clone())


def slice_inplace(self, ax: int, start: int, stop: int, step: int = 1):
    """Narrow one axis; bad arguments leave the tensor as it is (tensor.mojo:2807-2875)."""
    if self.dim() == 0 or not 0 <= ax < self.dim() or step == 0:
        return self.copy()
    key = [slice(None)] * self.dim()
    key[ax] = slice(start, stop, step)
    if step < 0:
        r = range(self.size(ax))[slice(start, stop, step)]
        out = _raw(self).index_select(ax, torch.tensor(list(r), dtype=torch.long))
    else:
        out = _raw(self)[tuple(key)]
    return _wrap(out)


def index_axis(self, axis: int, index: int):
    return _wrap(_raw(self).select(axis, index))


def squeeze_all(self):
    return _wrap(_raw(self).squeeze())


def squeeze_axis(self, axis: int):
    r = _raw(self)
    return _wrap(r.squeeze(axis) if r.dim() and r.size(axis) == 1 else r)


def get2(self, i: int, j: int):
    return _raw(self)[i, j].item()


def set2(self, i: int, j: int, v) -> None:
    _raw(self)[i, j] = v


def len_(self) -> int:
    return int(self.size(0)) if self.dim() else 1


def row(self, i: int):
    return _wrap(_raw(self)[i])


def cat(self, others=None, dim: int = 0):
    ts = list(self) if others is None and not isinstance(self, torch.Tensor) else [self] + list(others or [])
    return _wrap(torch.cat([_raw(t) for t in ts], dim))


def split_sizes(self, sizes: Sequence[int], dim: int = 0):
    return [_wrap(t) for t in torch.split(_raw(self), list(sizes), dim)]


def reshape_like(self, other):
    return _wrap(_raw(self).reshape(tuple(other.shape)))


def resize_like_with_pad(self, other, value=0):
    from .transform import resize_like_with_pad as f
    return f(self, other, value)


def can_broadcast_with(self, other, strict: bool = False) -> bool:
    from .broadcast import can_broadcast_shapes
    return can_broadcast_shapes(list(self.shape), list(other.shape), strict)


def fill(self, v) -> None:
    _raw(self).fill_(v)


# ---- storage builders (tensor.mojo:5566-5635) ---------------------------------------------------------------
def _grow(self, vals) -> None:
    n = self.numel()
    add = torch.as_tensor(vals, dtype=self.dtype).reshape(-1)
    if not self.is_contiguous():
        raise ValueError("append: the tensor must be dense")
    torch.Tensor.resize_(self, n + add.numel())
    _raw(self).view(-1)[n:] = add


def append(self, x) -> None:
    _grow(self, [x])


def append_list(self, xs) -> None:
    if len(xs):
        _grow(self, list(xs))


def append_repeat(self, val, count: int) -> None:
    if count > 0:
        _grow(self, [val] * count)


def append_strided(self, src, base: int, n: int, step: int = 1) -> None:
    if n > 0:
        _grow(self, [src[base + k * step] for k in range(n)])


def set_shape_row_major(self, shape: List[int]) -> None:
    """Give the appended storage its shape; the element count must match (tensor.mojo:5628-5634)."""
    torch.Tensor.resize_(self, tuple(int(s) for s in shape))


# ---- bitwise / shift / modulo spellings (tensor.mojo:4934-5241) ---------------------------------------------
def _i(x):
    r = _raw(x) if isinstance(x, torch.Tensor) else torch.as_tensor(x)
    return r.to(torch.int64)


def and_bitwise(self, o):
    return _wrap(_i(self) & _i(o))


def or_bitwise(self, o):
    return _wrap(_i(self) | _i(o))


def xor_bitwise(self, o):
    return _wrap(_i(self) ^ _i(o))


def not_bitwise(self):
    """0/1 integers: 1 where the element is zero (tensor.mojo:5241-5243)."""
    return _wrap((_raw(self) == 0).to(torch.int64))


and_scalar, or_scalar, xor_scalar = and_bitwise, or_bitwise, xor_bitwise


def lshift(self, o):
    return _wrap((_i(self) << _i(o)).to(self.dtype))


def rshift(self, o):
    return _wrap((_i(self) >> _i(o)).to(self.dtype))


lshift_scalar, rshift_scalar = lshift, rshift


def mod(self, o):
    from .math import mod_t
    return mod_t(self, o if isinstance(o, torch.Tensor) else _wrap(torch.as_tensor(o, dtype=self.dtype)))


mod_scalar = mod


# ---- conversions and text (tensor.mojo:3325-3420, 5463-5473) -----------------------------------------------
def to_float32(self):
    return _wrap(_raw(self).to(torch.float32))


def to_float64(self):
    return _wrap(_raw(self).to(torch.float64))


def to_int(self):
    return _wrap(_raw(self).to(torch.int64))


astype_float32, astype_float64 = to_float32, to_float64


def to_string(self) -> str:
    from .printing import tensor_to_string
    return tensor_to_string(self)


def dump(self) -> None:
    print(to_string(self))


# ---- integer set operations (tensor.mojo:3425-3520): sorted unique values -----------------------------------
def set_union(self, o):
    return _wrap(torch.unique(torch.cat([_raw(self).reshape(-1), _raw(o).reshape(-1)])))


def set_intersection(self, o):
    a, b = torch.unique(_raw(self)), torch.unique(_raw(o))
    return _wrap(a[torch.isin(a, b)])


def set_difference(self, o):
    a, b = torch.unique(_raw(self)), torch.unique(_raw(o))
    return _wrap(a[~torch.isin(a, b)])


def set_xor(self, o):
    a, b = torch.unique(_raw(self)), torch.unique(_raw(o))
    return _wrap(torch.cat([a[~torch.isin(a, b)], b[~torch.isin(b, a)]]).sort().values)


_METHODS = dict(
    idx=idx, slc=slc, all_axis=all_axis, rng=rng, reange=reange, full=full, pad_full_axes=pad_full_axes,
    select_view=select_view, select_copy=select_copy, select_set_scalar=select_set_scalar,
    select_set_tensor=select_set_tensor, slice=slice_, slice_inplace=slice_inplace, index_axis=index_axis,
    squeeze_all=squeeze_all, squeeze_axis=squeeze_axis, get2=get2, set2=set2, len=len_, row=row, cat=cat,
    split_sizes=split_sizes, reshape_like=reshape_like, resize_like_with_pad=resize_like_with_pad,
    can_broadcast_with=can_broadcast_with, fill=fill, append=append, append_list=append_list,
    append_repeat=append_repeat, append_strided=append_strided, set_shape_row_major=set_shape_row_major,
    and_bitwise=and_bitwise, or_bitwise=or_bitwise, xor_bitwise=xor_bitwise, not_bitwise=not_bitwise,
    and_scalar=and_scalar, or_scalar=or_scalar, xor_scalar=xor_scalar, lshift=lshift, rshift=rshift,
    lshift_scalar=lshift_scalar, rshift_scalar=rshift_scalar, mod=mod, mod_scalar=mod_scalar,
    to_float32=to_float32, to_float64=to_float64, to_int=to_int, astype_float32=astype_float32,
    astype_float64=astype_float64, to_string=to_string, dump=dump, set_union=set_union,
    set_intersection=set_intersection, set_difference=set_difference, set_xor=set_xor)

for _name, _fn in _METHODS.items():
    if _name == "select" or _name not in Tensor.__dict__:
        setattr(Tensor, _name, _fn)
