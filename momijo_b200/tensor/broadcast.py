"""NumPy broadcasting, ``clip/clamp``, ``compare`` and ``matmul`` / ``tensordot``
(legacy/src/momijo/tensor/broadcast.mojo:123-1694). ``matmul`` supports 2-D x 1-D and 2-D x 2-D
like the reference (anything else raises; lenient mode returns an empty tensor). On CUDA bf16
operands the product runs on the tcgen05 GEMM kernel."""
from __future__ import annotations

import torch

from .errors import ErrorKind, Status, TensorError, check_broadcastable, raise_or
from .tensor import _raw, _wrap


def broadcast_shapes(a, b):
    st = check_broadcastable(a, b)
    if not st.ok:
        raise TensorError(st.kind, st.msg)
    return list(torch.broadcast_shapes(tuple(a), tuple(b)))


def broadcast_to(x, shape):
    return _wrap(torch.broadcast_to(_raw(x), list(shape)))


def can_broadcast(a, b) -> bool:
    return check_broadcastable(a, b).ok


def clip(x, lo=None, hi=None):
    return _wrap(torch.clamp(_raw(x), lo, hi))


clamp = clip


def compare(a, b, op="eq", mode: int = None):
    """``compare(a, b, "lt")`` returns the 0/1 mask; the reference's ``compare(a, b, out_mask, mode)`` writes it into
    ``out_mask`` (mode 0..5 = eq, ne, lt, le, gt, ge; legacy/src/momijo/tensor/broadcast.mojo:1232)."""
    if mode is not None:
        return compare_float32(a, b, op, mode)
    f = {"eq": torch.eq, "ne": torch.ne, "lt": torch.lt, "le": torch.le, "gt": torch.gt, "ge": torch.ge}[op]
    return _wrap(f(_raw(a), _raw(b) if isinstance(b, torch.Tensor) else b).to(torch.int64))


def matmul(a, b):
    a, b = _raw(a), _raw(b)
    ok = a.dim() == 2 and b.dim() in (1, 2) and a.shape[1] == b.shape[0]
    if not ok:
        fb = raise_or(Status.fail(ErrorKind.SHAPE, f"matmul {tuple(a.shape)} x {tuple(b.shape)}"),
                      torch.zeros(0, dtype=a.dtype))
        return _wrap(fb)
    if not a.dtype.is_floating_point and not b.dtype.is_floating_point:
        a, b = a.float(), b.float()  # Int @ Int -> Float32
    elif a.dtype != b.dtype:
        dt = torch.result_type(a, b)     # mixed operands meet at the promoted type
        a, b = a.to(dt), b.to(dt)
    if (a.is_cuda and a.dtype == torch.bfloat16 and b.dim() == 2 and b.dtype == torch.bfloat16
            and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0):
        from .. import ops

        return _wrap(ops.gemm(a, b, b_mn=True))
    return _wrap(a @ b)


def tensordot(a, b, axes: int = 1):
    return _wrap(torch.tensordot(_raw(a), _raw(b), dims=axes))


# ---- further broadcasting names of the reference (legacy/src/momijo/tensor/broadcast.mojo:42-1990) ------------------
# Out-parameter kernels (``add_(a, b, out)`` ...) write into ``out`` in place. Scalar op tables:
# bin32 / bin64: 0 add, 1 sub, 2 mul, 3 div, 4 pow (0 for a non-positive base), 5 min, anything else max;
# u32 / u64: 0 neg, 1 abs, 2 exp, 3 log, 4 sqrt, 5 tanh, 6 relu, anything else expm1;
# cmp32 / cmp64: 0 eq, 1 ne, 2 lt, 3 le, 4 gt, 5 ge.
import math as _math  # noqa: E402
from dataclasses import dataclass as _dataclass, field as _field  # noqa: E402


def pad_left_ones(x, r: int):
    x = list(x)
    return [1] * max(r - len(x), 0) + x


def align_right(a, b):
    r = max(len(a), len(b))
    return pad_left_ones(a, r), pad_left_ones(b, r)


def same_shape(a, b) -> bool:
    return list(a) == list(b)


def can_broadcast_shapes(a, b, strict: bool = False) -> bool:
    """NumPy rule (right-aligned, missing axes count as 1); ``strict`` also wants equal rank
    (legacy/src/momijo/tensor/broadcast.mojo:2012-2080)."""
    if strict and len(a) != len(b):
        return False
    pa, pb = align_right(a, b)
    return all(x == y or x == 1 or y == 1 for x, y in zip(pa, pb))


can_broadcast_shapes_numpy = can_broadcast_shapes


def can_broadcast_shapes_strict(a, b) -> bool:
    """Same rank required; each axis equal or 1."""
    return len(a) == len(b) and can_broadcast_shapes(a, b)


def broadcast_shapes_many(shapes, out_shape: list = None):
    """Common broadcast shape of several shapes: returns (ok, shape) and also fills ``out_shape`` if given."""
    acc: list = []
    ok = True
    for s in shapes:
        if not can_broadcast_shapes(acc, s):
            ok, acc = False, []
            break
        pa, pb = align_right(acc, s)
        acc = [max(x, y) for x, y in zip(pa, pb)]
    if out_shape is not None:
        out_shape[:] = acc
    return ok, acc


@_dataclass
class BroadcastResult:
    ok: bool = False
    shape: list = _field(default_factory=list)
    lhs_padded: list = _field(default_factory=list)
    rhs_padded: list = _field(default_factory=list)
    lhs_strides: list = _field(default_factory=list)
    rhs_strides: list = _field(default_factory=list)


def broadcast_batch_strides(in_shape, in_strides, out_shape):
    """Strides of ``in_shape`` viewed as ``out_shape``: 0 on broadcast (extent 1 or missing) axes."""
    ps = pad_left_ones(in_shape, len(out_shape))
    st = [0] * (len(out_shape) - len(in_strides)) + list(in_strides)
    return [0 if d == 1 and o != 1 else s for d, s, o in zip(ps, st, out_shape)]


def prepare_broadcast(lhs_shape, lhs_strides, rhs_shape, rhs_strides):
    ok, shape = broadcast_shapes_many([lhs_shape, rhs_shape])
    if not ok:
        return False, BroadcastResult()
    pl, pr = align_right(lhs_shape, rhs_shape)
    return True, BroadcastResult(True, shape, pl, pr, broadcast_batch_strides(lhs_shape, lhs_strides, shape),
                                 broadcast_batch_strides(rhs_shape, rhs_strides, shape))


def broadcast_like(x, other):
    return _wrap(_raw(x).expand(_raw(other).shape))


def keepdims_shape(shape, axes):
    """Shape after reducing ``axes`` with keepdims: those extents become 1."""
    r = len(shape)
    ax = {a + r if a < 0 else a for a in axes}
    return [1 if i in ax else d for i, d in enumerate(shape)]


def clamp_f64(x, lo, hi): return lo if x < lo else (hi if x > hi else x)      # noqa: E704


clamp_int = clamp_f64


def clamp_axis(ax: int, rank: int) -> int:
    v = ax + rank if ax < 0 else ax
    return min(max(v, 0), max(rank - 1, 0))


def tanh64(x: float) -> float: return _math.tanh(x)       # noqa: E704


def bin64(x: float, y: float, op: int) -> float:
    if op == 0:
        return x + y
    if op == 1:
        return x - y
    if op == 2:
        return x * y
    if op == 3:
        return x / y if y != 0 else _math.copysign(_math.inf, x) if x != 0 else _math.nan
    if op == 4:
        return 0.0 if x <= 0.0 else _math.exp(y * _math.log(x))
    return min(x, y) if op == 5 else max(x, y)


def u64(x: float, op: int) -> float:
    if op == 0:
        return -x
    if op == 1:
        return abs(x)
    if op == 2:
        return _math.exp(x)
    if op == 3:
        return _math.log(x) if x > 0 else (-_math.inf if x == 0 else _math.nan)
    if op == 4:
        return _math.sqrt(x) if x >= 0 else _math.nan
    if op == 5:
        return _math.tanh(x)
    if op == 6:
        return x if x > 0 else 0.0
    return _math.expm1(x)


def _r32(v):
    from .scalar_cast import _to_f32
    return _to_f32(v)


def bin32(x, y, op): return _r32(bin64(_r32(x), _r32(y), op))       # noqa: E704
def u32(x, op): return _r32(u64(_r32(x), op))                       # noqa: E704


def cmp64(a, b, m: int) -> int:
    return int([a == b, a != b, a < b, a <= b, a > b, a >= b][m if 0 <= m <= 5 else 5])


cmp32 = cmp64


def ipow_generic(base, exp_i: int):
    """Integer power by squaring (negative exponents give 1, as the loop never runs)."""
    res, b, e = type(base)(1), base, exp_i
    while e > 0:
        if e & 1:
            res = res * b
        b = b * b
        e >>= 1
    return res


def pow_generic_safe(x, y_val):
    """x ** int(y) for non-float element types; a zero exponent gives 1, a negative one 0 unless x is 1 or -1."""
    iy = int(y_val)
    if iy == 0:
        return type(x)(1)
    if iy < 0:
        return x if x == 1 else (type(x)(1 if iy % 2 == 0 else -1) if x == -1 else type(x)(0))
    return ipow_generic(x, iy)


_BIN = {0: torch.add, 1: torch.sub, 2: torch.mul, 3: torch.div, 4: torch.pow, 5: torch.minimum}


def apply_broadcast_binary(a, b, out, op: int) -> None:
    o = _raw(out)
    r = _BIN.get(op, torch.maximum)(_raw(a), _raw(b))
    o.copy_(r.to(o.dtype))


apply_broadcast_binary_float32 = apply_broadcast_binary_float64 = apply_broadcast_binary


def add_(a, b, out): apply_broadcast_binary(a, b, out, 0)          # noqa: E704
def sub_(a, b, out): apply_broadcast_binary(a, b, out, 1)          # noqa: E704
def mul_(a, b, out): apply_broadcast_binary(a, b, out, 2)          # noqa: E704
def div_(a, b, out): apply_broadcast_binary(a, b, out, 3)          # noqa: E704
def pow_(a, b, out): apply_broadcast_binary(a, b, out, 4)          # noqa: E704
def minimum_(a, b, out): apply_broadcast_binary(a, b, out, 5)      # noqa: E704
def maximum_(a, b, out): apply_broadcast_binary(a, b, out, 6)      # noqa: E704


_UN = {0: torch.neg, 1: torch.abs, 2: torch.exp, 3: torch.log, 4: torch.sqrt, 5: torch.tanh,
       6: lambda t: t.clamp_min(0)}


def apply_unary(x, out, op: int) -> None:
    o = _raw(out)
    o.copy_(_UN.get(op, torch.expm1)(_raw(x)).to(o.dtype))


apply_unary_float32 = apply_unary_float64 = apply_unary


def sign_(x, out) -> None:
    o = _raw(out)
    o.copy_(torch.sign(_raw(x)).to(o.dtype))


sign_float32 = sign_float64 = sign_


def compare_float32(a, b, out_mask, mode: int) -> None:
    """Element-wise comparison (mode as in ``cmp32``) written into an integer mask in place."""
    ta, tb = _raw(a), _raw(b)
    r = [ta == tb, ta != tb, ta < tb, ta <= tb, ta > tb, ta >= tb][mode if 0 <= mode <= 5 else 5]
    o = _raw(out_mask)
    o.copy_(r.to(o.dtype))


compare_float64 = compare_float32


def matmul_core_vec(A, x):
    a, v = _raw(A), _raw(x)
    if a.dim() != 2 or v.dim() != 1 or a.shape[1] != v.shape[0]:
        return _wrap(torch.zeros(0, dtype=a.dtype))
    return _wrap(a @ v)


def matmul_core_mm(A, B):
    a, b = _raw(A), _raw(B)
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        return _wrap(torch.zeros(0, dtype=a.dtype))
    return matmul(_wrap(a), _wrap(b))
