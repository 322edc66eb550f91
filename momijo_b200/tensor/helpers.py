"""Stride / contiguity / selector helpers (legacy/src/momijo/tensor/helpers.mojo)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .tensor import _raw, _wrap


def compute_row_major_strides(shape) -> List[int]:
    s, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        s[i] = acc
        acc *= max(int(shape[i]), 1)
    return s


mk_strides = compute_row_major_strides


def is_contiguous(shape, strides, row_major: bool = True) -> bool:
    """Strides of a dense layout: row-major, or column-major with ``row_major=False``
    (legacy/src/momijo/tensor/helpers.mojo:841-860)."""
    if row_major:
        return list(strides) == compute_row_major_strides(shape)
    exp, acc = [], 1
    for d in shape:
        exp.append(acc)
        acc *= d
    return list(strides) == exp


def numel(shape) -> int:
    n = 1
    for v in shape:
        n *= int(v)
    return n


@dataclass
class SliceSpec:
    start: Optional[int] = None
    stop: Optional[int] = None
    step: Optional[int] = None

    def to_slice(self):
        return slice(self.start, self.stop, self.step)


@dataclass
class IndexSel:
    """One selector: an integer index, a slice, or a list of indices (fancy)."""
    index: Optional[int] = None
    slice: Optional[SliceSpec] = None
    fancy: Optional[List[int]] = None

    def to_key(self):
        if self.index is not None:
            return self.index
        if self.fancy is not None:
            return list(self.fancy)
        return (self.slice or SliceSpec()).to_slice()


def normalize_slice_1d(n: int, start, stop, step):
    """Python slice normalisation including negative steps."""
    return slice(start, stop, step).indices(n)


def select(x, sels: List[IndexSel]):
    return _wrap(_raw(x)[tuple(s.to_key() for s in sels)])


def write_plane(x, axis: int, index: int, plane):
    """x.select(axis, index) = plane (in place); returns x."""
    _raw(x).select(axis, index).copy_(_raw(plane))
    return x


write_planeT = write_plane      # the reference spells one overload this way (legacy/src/momijo/tensor/helpers.mojo:753)


class XorShift64:
    def __init__(self, seed: int = 88172645463325252):
        self.s = (seed or 88172645463325252) & ((1 << 64) - 1)

    def next_u64(self) -> int:
        x = self.s
        x ^= (x << 13) & ((1 << 64) - 1)
        x ^= x >> 7
        x ^= (x << 17) & ((1 << 64) - 1)
        self.s = x
        return x

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)

    next_unit_f64 = uniform


def sort_values(x, descending=False):
    return _wrap(torch.sort(_raw(x).reshape(-1), descending=descending, stable=True).values)


def argsort_values(x, descending=False):
    return _wrap(torch.argsort(_raw(x).reshape(-1), descending=descending, stable=True))


def unique_values(x):
    return _wrap(torch.unique(_raw(x)))


# ---- further helper names of the reference (legacy/src/momijo/tensor/helpers.mojo:60-3760) ---------------------------
# Shapes, strides and index arithmetic work on plain lists; sorting / set operations accept lists or
# tensors and return the same kind; selector constructors build the ``IndexSel`` / ``SliceSpec`` above.
import bisect as _bisect  # noqa: E402

import torch as _torch  # noqa: E402


def _is_tensor(x):
    return isinstance(x, _torch.Tensor) or hasattr(x, "shape") and not isinstance(x, (list, tuple))


def _flat_list(x):
    return _raw(x).reshape(-1).tolist() if _is_tensor(x) else list(x)


def numel_shape(shape) -> int: return numel(shape)                                       # noqa: E704
def row_major_strides(shape): return compute_row_major_strides(shape)                    # noqa: E704
def make_strides_row_major(shape): return compute_row_major_strides(shape)               # noqa: E704
def strides_for_shape(shape): return compute_row_major_strides(shape)                    # noqa: E704
def ensure_strides(shape, strides=None): return list(strides) if strides else compute_row_major_strides(shape)  # noqa: E704,E501
def identity_perm(n: int): return list(range(n))                                         # noqa: E704
def same_shape(a, b) -> bool: return list(getattr(a, "shape", a)) == list(getattr(b, "shape", b))   # noqa: E704
def lists_equal_int(a, b) -> bool: return list(a) == list(b)                             # noqa: E704
def min_i(a: int, b: int) -> int: return a if a < b else b                               # noqa: E704
def max_i(a: int, b: int) -> int: return a if a > b else b                               # noqa: E704
def clamp_nonneg(x: int) -> int: return x if x > 0 else 0                                # noqa: E704
def ceil_div_pos(a: int, b: int) -> int: return (a + b - 1) // b if b > 0 else 0         # noqa: E704
def reserve_len(xs, n: int = None):
    """``reserve_len(n)`` clamps a length at 0; the reference's ``reserve_len(list, n)`` appends ``n`` zeros to the list
    in place (legacy/src/momijo/tensor/helpers.mojo:114-120)."""
    if n is None:
        return max(xs, 0)
    xs.extend([0] * max(n, 0))
def copy_list(xs): return list(xs)                                                       # noqa: E704


copy_list_T = copy_list_int = copy_ints = copy_list


def copy_flat_list(x): return _flat_list(x)             # noqa: E704


setops_copy_flat_list = copy_flat_list


def tolist(x, f=None):
    """Flat list of the elements, each passed through ``f`` (the reference's converter to Float64) when given."""
    vals = copy_flat_list(x)
    return [f(v) for v in vals] if f is not None else vals


# ``f`` is the reference's per-element converter; without it the built-in conversion is used.
def to_int_list(x, f=None): return [(f or int)(v) for v in _flat_list(x)]        # noqa: E704
def to_bool_list(x, f=None): return [(f or bool)(v) for v in _flat_list(x)]      # noqa: E704
def tensor_len(x) -> int: return _raw(x).numel()                  # noqa: E704
def size(x) -> int: return _raw(x).numel() if _is_tensor(x) else len(x)   # noqa: E704
def dim0_length(x) -> int: return int(_raw(x).shape[0]) if _raw(x).dim() else 1   # noqa: E704
def tensor1d_from_list(xs, dtype=None): return _wrap(_torch.tensor(list(xs), dtype=dtype))   # noqa: E704
def tensor_sum_float(x) -> float: return float(_raw(x).double().sum())    # noqa: E704
def tensor_sum_int(x) -> int: return int(_raw(x).sum())                   # noqa: E704
def scalar_UInt8(v): return _wrap(_torch.tensor(int(v) & 255, dtype=_torch.uint8))    # noqa: E704
def scalar_int32(v): return _wrap(_torch.tensor(int(v), dtype=_torch.int32))          # noqa: E704
def scalar_int64(v): return _wrap(_torch.tensor(int(v), dtype=_torch.int64))          # noqa: E704
def one_scalar_of(from_f64): return from_f64(1.0)                                     # noqa: E704
def zero_scalar_of(from_f64): return from_f64(0.0)                                    # noqa: E704
def f64_of_f32(v): return float(v)                                                    # noqa: E704


f64_of_f64 = f64_of_int = f64_of_f32


def int_of_f32(v): return int(v)      # noqa: E704


int_of_f64 = int_of_int = int_of_f32


def bool_of_f32(v): return v != 0     # noqa: E704


bool_of_f64 = bool_of_int = bool_of_f32


def eq_f64(a, b): return a == b       # noqa: E704
def lt_f64(a, b): return a < b        # noqa: E704


eq_int, lt_int = eq_f64, lt_f64


def normalize_axis(axis: int, rank: int) -> int:
    """Negative axes count from the end; the result is clamped into [0, rank - 1]."""
    a = axis + rank if axis < 0 else axis
    return min(max(a, 0), max(rank - 1, 0))


def wrap_index(i: int, dim: int) -> int:
    return i + dim if i < 0 else i


def wrap_axis_index(i: int, dim: int) -> int:
    return min(max(wrap_index(i, dim), 0), max(dim - 1, 0))


def range_len(start: int, stop: int, step: int) -> int:
    step = step or 1
    n = (stop - start + (step - (1 if step > 0 else -1))) // step
    return max(n, 0)


axis_len_from_slice = range_len


def shape_drop_axis(shape, axis: int):
    a = normalize_axis(axis, len(shape))
    return [d for i, d in enumerate(shape) if i != a]


def lin_index(idx, strides) -> int:
    return sum(int(i) * int(s) for i, s in zip(idx, strides))


flat_index = lin_index


def flat_index_bcast(idx, shape, strides) -> int:
    """Linear offset where axes of extent 1 are broadcast (their index is ignored)."""
    return sum((0 if d == 1 else int(i)) * int(s) for i, d, s in zip(idx, shape, strides))


def unravel_index(lin: int, shape, out_idx=None):
    idx = []
    for d in reversed(list(shape)):
        idx.append(lin % d if d > 0 else 0)
        lin //= d if d > 0 else 1
    idx.reverse()
    if out_idx is not None:
        out_idx[:] = idx
    return idx


def index_advance(idx, shape) -> bool:
    """Odometer step over ``shape`` (last axis fastest), in place; False after the last position."""
    for ax in range(len(shape) - 1, -1, -1):
        idx[ax] += 1
        if idx[ax] < shape[ax]:
            return True
        idx[ax] = 0
    return False


def compute_new_shape(old_shape, pad_pairs):
    return [int(d) + int(lo) + int(hi) for d, (lo, hi) in zip(old_shape, pad_pairs)]


def ensure_2d(x):
    """Scalars and vectors become [1, n]; higher ranks collapse their leading axes."""
    t = _raw(x)
    return x if t.dim() == 2 else _wrap(t.reshape(1, -1) if t.dim() < 2 else t.reshape(-1, t.shape[-1]))


def ensure_4d(x):
    t = _raw(x)
    if t.dim() == 4:
        return x
    if t.dim() > 4:
        return _wrap(t.reshape(-1, *t.shape[-3:]))
    return _wrap(t.reshape((1,) * (4 - t.dim()) + tuple(t.shape)))


def is_contiguous_tensor(x) -> bool: return _raw(x).is_contiguous()         # noqa: E704


def is_row_major_contiguous(x, strides=None) -> bool:
    """A tensor, or the reference's ``(shape, strides)`` pair (legacy/src/momijo/tensor/helpers.mojo:274-286)."""
    return is_contiguous_tensor(x) if strides is None else is_contiguous(list(x), list(strides))


def is_contig_2d(x, width: int = None) -> bool:
    """A 2-D tensor, or the reference's ``(strides, width)``: strides equal to ``[width, 1]``
    (legacy/src/momijo/tensor/helpers.mojo:288-291)."""
    if width is not None:
        return list(x) == [width, 1]
    t = _raw(x)
    return t.dim() == 2 and t.is_contiguous()


def maybe_copy(x):
    """The tensor itself when it is contiguous, else a packed copy."""
    t = _raw(x)
    return x if t.is_contiguous() else _wrap(t.contiguous())


def clone_header_share_data(x, shape, strides):
    """New view of the same storage with the given shape and element strides."""
    return _wrap(_torch.as_strided(_raw(x), list(shape), list(strides)))


def astype_with(src, f):
    t = _raw(src)
    return _wrap(_torch.tensor([f(v) for v in t.reshape(-1).tolist()]).reshape(t.shape))


def astype_float64(x): return _wrap(_raw(x).double())       # noqa: E704


def astype_via_f64(src, to_f64=None, from_f64=None):
    """Convert element by element through float64: ``from_f64(to_f64(v))`` (legacy/src/momijo/tensor/helpers.mojo:
    973-1010). Without converters this is the float64 cast."""
    if to_f64 is None and from_f64 is None:
        return astype_float64(src)
    r = _raw(src)
    vals = [(from_f64 or float)((to_f64 or float)(v)) for v in r.reshape(-1).tolist()]
    return _wrap(_torch.tensor(vals).reshape(list(r.shape)))


def apply_bin_f32(a, b, op_id: int):
    from .math_compat import apply_broadcast2
    return apply_broadcast2(a, b, op_id)


apply_bin_f64 = apply_bin_Int32 = apply_bin_Int64 = apply_bin_f32


def apply_cmp_f32(a, b, mode: int):
    """Element-wise comparison as uint8 0/1: 0 eq, 1 ne, 2 lt, 3 le, 4 gt, 5 ge."""
    ta, tb = _raw(a), _raw(b) if _is_tensor(b) else b
    r = [ta == tb, ta != tb, ta < tb, ta <= tb, ta > tb, ta >= tb][mode if 0 <= mode <= 5 else 5]
    return _wrap(r.to(_torch.uint8))


apply_cmp_f64 = apply_cmp_Int = apply_cmp_Int32 = apply_cmp_Int64 = apply_cmp_UInt8 = apply_cmp_f32


# ---- selectors ----
def make_slice(start: int, stop: int, step: int = 1) -> SliceSpec: return SliceSpec(start, stop, step)   # noqa: E704
def full_axis_slice(dim: int) -> SliceSpec: return SliceSpec(0, dim, 1)                                  # noqa: E704
def full_axis(dim: int) -> IndexSel: return IndexSel(slice=SliceSpec(0, dim, 1))                         # noqa: E704
def make_index_sel(i: int) -> IndexSel: return IndexSel(index=i)                                         # noqa: E704
def make_fancy_sel(js) -> IndexSel: return IndexSel(fancy=list(js))                                      # noqa: E704


def make_slice_sel(start, stop=None, step=None) -> IndexSel:
    if isinstance(start, tuple):
        start, stop, step = start
    return IndexSel(slice=SliceSpec(start, stop, step))


sel_index, sel_slice = make_index_sel, make_slice_sel


def is_index(s: IndexSel) -> bool: return s.index is not None                     # noqa: E704
def is_fancy(s: IndexSel) -> bool: return s.index is None and s.fancy is not None  # noqa: E704
def is_slice(s: IndexSel) -> bool: return s.index is None and s.fancy is None      # noqa: E704


sel_is_index = is_index


def get_index(s: IndexSel) -> int: return s.index                                  # noqa: E704
def get_fancy_list(s: IndexSel): return list(s.fancy or [])                         # noqa: E704


def get_slice(s: IndexSel):
    sp = s.slice or SliceSpec()
    return sp.start, sp.stop, sp.step


# ---- sorting and set operations ----
def insertion_sort(xs):
    """Sorted copy (stable)."""
    return sorted(xs)


def insertion_sort_inplace(xs):
    xs.sort()
    return xs


setops_insertion_sort_f64 = setops_insertion_sort_int = insertion_sort


def _sort(x, descending=False):
    if _is_tensor(x):
        return _wrap(_torch.sort(_raw(x).reshape(-1), descending=descending, stable=True).values)
    return sorted(x, reverse=descending)


def _argsort(x, descending=False):
    if _is_tensor(x):
        return _wrap(_torch.argsort(_raw(x).reshape(-1), descending=descending, stable=True))
    return sorted(range(len(x)), key=lambda i: x[i], reverse=descending)


sort_f32 = sort_f64 = sort_int = tensor_sort_f32 = tensor_sort_f64 = tensor_sort_int = _sort
argsort_f32 = argsort_f64 = argsort_int = _argsort


def unique_from_sorted(xs):
    out = []
    for v in xs:
        if not out or out[-1] != v:
            out.append(v)
    return out


setops_unique_from_sorted_f64 = setops_unique_from_sorted_int = unique_from_sorted


def sorted_unique(xs):
    return unique_from_sorted(sorted(_flat_list(xs)))


setops_sorted_unique_f64 = setops_sorted_unique_int = sorted_unique


class UniqueResult:
    """Sorted distinct values and how often each occurs."""

    def __init__(self, values, counts):
        self.values, self.counts = values, counts


def unique(x, return_counts: bool = True) -> UniqueResult:
    """Sorted distinct values; the counts are empty when ``return_counts`` is false."""
    vals, counts = _torch.unique(_raw(x).reshape(-1), sorted=True, return_counts=True)
    return UniqueResult(_wrap(vals), _wrap(counts if return_counts else counts[:0]))


unique_int = unique_float32 = unique_float64 = tensor_unique_int = tensor_unique_f32 = tensor_unique_f64 = unique


def bincount_int(x):
    """Counts of the non-negative integers 0..max (negative entries are ignored)."""
    t = _raw(x).reshape(-1).long()
    t = t[t >= 0]
    return _wrap(_torch.bincount(t) if t.numel() else _torch.zeros(0, dtype=_torch.int64))


tensor_bincount_int = bincount_int


def histogram_int(x, bins) -> UniqueResult:
    """Counts per half-open bin [bins[i], bins[i+1]) (the last bin also takes its right edge); ``values`` holds the
    left edges. Fewer than two edges give empty results."""
    edges = list(bins)
    if len(edges) < 2:
        z = _torch.zeros(0, dtype=_torch.int64)
        return UniqueResult(_wrap(z), _wrap(z.clone()))
    counts = [0] * (len(edges) - 1)
    for v in _flat_list(x):
        if edges[0] <= v <= edges[-1]:
            counts[min(_bisect.bisect_right(edges, v) - 1, len(counts) - 1)] += 1
    return UniqueResult(_wrap(_torch.tensor(edges[:-1])), _wrap(_torch.tensor(counts)))


tensor_histogram_int = histogram_int


def digitize_int(x, edges):
    """Index of the bin each value falls in: number of edges <= value."""
    e = list(edges)
    t = _raw(x)
    return _wrap(_torch.tensor([_bisect.bisect_right(e, v) for v in t.reshape(-1).tolist()]).reshape(t.shape))


tensor_digitize_int = digitize_int


# ---- small text helpers ----
def trim_ascii(s: str) -> str: return s.strip(" \t\r\n")          # noqa: E704


def digit_from_one_char(ch: str) -> int:
    return ord(ch) - 48 if len(ch) == 1 and "0" <= ch <= "9" else -1


def parse_int_safe(s: str, default: int = 0) -> int:
    try:
        return int(trim_ascii(s))
    except ValueError:
        return default


def to_string_owned(x) -> str: return str(x)                       # noqa: E704


def tensor_to_string_core(x) -> str:
    from .cast import to_string
    return to_string(x)


def uniform_f32(rng, low: float = 0.0, high: float = 1.0) -> float:
    """One draw from ``rng`` (anything with ``next_u64``, e.g. ``XorShift64``) mapped to [low, high)."""
    u = (rng.next_u64() >> 11) / 9007199254740992.0
    return low + (high - low) * u


def append_block_unrolled16(dst: list, src, src_lo: int, src_hi: int) -> None:
    dst.extend(src[src_lo:src_hi])


def append_repeat_unrolled8(dst: list, v, count: int) -> None:
    dst.extend([v] * max(count, 0))
