"""Scalar math shims, op-id dispatchers, logical and in-place tensor ops of the reference's math module
(legacy/src/momijo/tensor/math.mojo:41-3950).

Scalar functions come in ``*32`` / ``*64`` pairs (the 32-bit ones round their result to float32). The
dispatchers take the reference's numeric op ids:

* unary (``apply_unary``): 0 neg, 1 abs, 2 sqrt, 3 exp, 4 log, 5 sin, 6 cos, 7 tan, 8 relu, 9 expm1, 10 log1p,
  11 floor, 12 ceil, 13 round (half away from zero), 14 sign, 15 sigmoid, 16 tanh, 17 silu, 18 gelu (tanh form),
  19 elu, 20 selu; integer inputs are promoted to float64;
* binary (``apply_broadcast2`` .. ``5``): 0 add, 1 sub, 2 mul, 3 div, 4 pow, 5 max, 6 min, 7 mod,
  10/20 and, 11/21 or, 12/22 xor, 13/23 nand, 14/24 nor, 15/25 xnor, 16/26 andnot; ids 10-16 return 0/1 integers,
  ids 20-26 booleans;
* compare (``cmp_eval``): 0 eq, 1 ne, 2 lt, 3 le, 4 gt, 5 ge."""
from __future__ import annotations

import math
import struct

import torch

from .tensor import _raw, _wrap


def _f32(v: float) -> float:
    try:
        return struct.unpack("<f", struct.pack("<f", float(v)))[0]
    except OverflowError:
        return math.copysign(math.inf, v)


def abs64(x): return -x if x < 0 else x                                 # noqa: E704
def sqrt64(x): return math.sqrt(x) if x > 0 else 0.0                    # noqa: E704
def exp64(x): return math.exp(x) if x < 709.0 else math.inf             # noqa: E704
def log64(x): return math.log(x) if x > 0 else (-math.inf if x == 0 else math.nan)   # noqa: E704
def sin64(x): return math.sin(x)                                        # noqa: E704
def cos64(x): return math.cos(x)                                        # noqa: E704
def tan64(x): return math.tan(x)                                        # noqa: E704
def tanh64(x): return math.tanh(x)                                      # noqa: E704
def expm1_64(x): return math.expm1(x) if x < 709.0 else math.inf        # noqa: E704
def log1p64(x): return math.log1p(x) if x > -1 else (-math.inf if x == -1 else math.nan)   # noqa: E704
def floor64(x): return float(math.floor(x))                             # noqa: E704
def ceil64(x): return float(math.ceil(x))                               # noqa: E704
def round64(x): return floor64(x + 0.5) if x >= 0 else ceil64(x - 0.5)  # noqa: E704
def sign64(x): return 1.0 if x > 0 else (-1.0 if x < 0 else 0.0)        # noqa: E704
def sigmoid64(x): return 1.0 / (1.0 + math.exp(-x)) if x >= 0 else math.exp(x) / (1.0 + math.exp(x))   # noqa: E704
def silu64(x): return x * sigmoid64(x)                                  # noqa: E704
def gelu64(x): return 0.5 * x * (1.0 + math.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))   # noqa: E704
def elu64(x): return x if x >= 0 else math.expm1(x)                     # noqa: E704
def selu64(x): return 1.0507009873554804 * (x if x >= 0 else 1.6732632423543772 * math.expm1(x))   # noqa: E704
def pow64(a, b): return float(a) ** float(b)                            # noqa: E704


for _n in ("abs", "sqrt", "exp", "log", "sin", "cos", "tan", "tanh", "floor", "ceil", "round", "sign", "sigmoid",
           "silu", "gelu", "elu", "selu"):
    globals()[f"{_n}32"] = (lambda f: (lambda x: _f32(f(x))))(globals()[f"{_n}64"])
expm1_32 = lambda x: _f32(expm1_64(x))      # noqa: E731
log1p32 = lambda x: _f32(log1p64(x))        # noqa: E731
pow32 = lambda a, b: _f32(pow64(a, b))      # noqa: E731


def safe_div32(a: float, b: float, eps: float = 1e-7) -> float:
    """a / (b + eps) with the bias taking the sign of ``b`` (zero counts as positive)."""
    return _f32(a / (b + eps if b >= 0 else b - eps))


def safe_sqrt32(x: float, eps: float = 0.0) -> float:
    """``sqrt(max(x, 0) + eps)`` in float32; the reference's default eps is 1e-7 (legacy/src/momijo/tensor/
    math.mojo:262-267), this package's stays 0 so that ``safe_sqrt32(0) == 0``."""
    v = max(x, 0.0) + eps
    return _f32(math.sqrt(v)) if v > 0 else 0.0


def math_max(a, b): return a if a >= b else b     # noqa: E704
def math_min(a, b): return a if a <= b else b     # noqa: E704


# ---- dispatchers ------------------------------------------------------------------------------------------------
def _rnd(t):
    return torch.where(t >= 0, (t + 0.5).floor(), (t - 0.5).ceil())


_UNARY = {
    0: torch.neg, 1: torch.abs, 2: lambda t: t.clamp_min(0).sqrt(), 3: torch.exp, 4: torch.log, 5: torch.sin,
    6: torch.cos, 7: torch.tan, 8: lambda t: t.clamp_min(0), 9: torch.expm1, 10: torch.log1p, 11: torch.floor,
    12: torch.ceil, 13: _rnd, 14: torch.sign, 15: torch.sigmoid, 16: torch.tanh, 17: torch.nn.functional.silu,
    18: lambda t: torch.nn.functional.gelu(t, approximate="tanh"), 19: torch.nn.functional.elu,
    20: torch.nn.functional.selu,
}


def apply_unary(x, uop_id: int):
    t = _raw(x)
    if not t.dtype.is_floating_point:
        t = t.double()
    return _wrap(_UNARY.get(uop_id, torch.sign)(t))


apply_unary_impl = apply_unary_impl32 = unary_eval_impl = unary_eval_impl32 = apply_unary


def _truth(t):
    return t != 0


def _binary(a, b, op_id: int):
    if op_id == 0:
        return a + b
    if op_id == 1:
        return a - b
    if op_id == 2:
        return a * b
    if op_id == 3:
        return a.double() / b.double() if not a.dtype.is_floating_point else a / b
    if op_id == 4:
        return torch.pow(a, b)
    if op_id == 5:
        return torch.maximum(a, b)
    if op_id == 6:
        return torch.minimum(a, b)
    if op_id == 7:
        return torch.remainder(a, b)
    k = op_id % 10
    p, q = _truth(a), _truth(b)
    r = {0: p & q, 1: p | q, 2: p ^ q, 3: ~(p & q), 4: ~(p | q), 5: ~(p ^ q), 6: p & ~q}[k]
    return r if op_id >= 20 else r.to(torch.int64)


def apply_broadcast2(a, b, op_id: int):
    ta, tb = _raw(a), _raw(b) if not isinstance(b, (int, float, bool)) else b
    if not isinstance(tb, torch.Tensor):
        tb = torch.tensor(tb, dtype=ta.dtype if isinstance(tb, float) == ta.dtype.is_floating_point else None)
    return _wrap(_binary(ta, tb, op_id))


apply_broadcast2_impl = apply_broadcast3 = apply_broadcast4 = apply_broadcast5 = bin_combine_impl = apply_broadcast2
elemwise2_same_contig_impl = apply_broadcast2


def elemwise_scalar_right_impl(x, s, op_id: int):
    return apply_broadcast2(x, s, op_id)


def elemwise_scalar_left_impl(s, x, op_id: int):
    t = _raw(x)
    return _wrap(_binary(torch.tensor(s, dtype=t.dtype if isinstance(s, float) == t.dtype.is_floating_point else None),
                         t, op_id))


def apply_broadcast2_inplace(x, y, op_id: int) -> None:
    """x <- x (op) y, keeping x's dtype and storage."""
    t = _raw(x)
    t.copy_(_binary(t, _raw(y) if not isinstance(y, (int, float)) else torch.tensor(y), op_id).to(t.dtype))


apply_broadcast2_inplace_impl = apply_broadcast2_inplace


def cmp_eval(a, b, mode: int) -> int:
    """Scalar comparison as 0 / 1."""
    return int([a == b, a != b, a < b, a <= b, a > b, a >= b][mode if 0 <= mode <= 5 else 5])


def iadd_t(x, y): apply_broadcast2_inplace(x, y, 0)           # noqa: E704
def isub_t(x, y): apply_broadcast2_inplace(x, y, 1)           # noqa: E704
def imul_t(x, y): apply_broadcast2_inplace(x, y, 2)           # noqa: E704
def idiv_t(x, y): apply_broadcast2_inplace(x, y, 3)           # noqa: E704
def imaximum_t(x, y): apply_broadcast2_inplace(x, y, 5)       # noqa: E704
def iminimum_t(x, y): apply_broadcast2_inplace(x, y, 6)       # noqa: E704


def ipow_scalar(x, p: float) -> None:
    t = _raw(x)
    t.copy_(torch.pow(t.double(), p).to(t.dtype))


def pow_scalar_right(x, p: float):
    return _wrap(torch.pow(_raw(x), p))


def pow_scalar_left(p: float, x):
    return _wrap(torch.pow(torch.tensor(float(p), dtype=torch.float64), _raw(x).double()).to(
        _raw(x).dtype if _raw(x).dtype.is_floating_point else torch.float64))


def mod_t(a, b): return apply_broadcast2(a, b, 7)             # noqa: E704
def nand_t(a, b): return apply_broadcast2(a, b, 13)           # noqa: E704
def nor_t(a, b): return apply_broadcast2(a, b, 14)            # noqa: E704
def xnor_t(a, b): return apply_broadcast2(a, b, 15)           # noqa: E704
def andnot_t(a, b): return apply_broadcast2(a, b, 16)         # noqa: E704
def land_t(a, b): return apply_broadcast2(a, b, 20)           # noqa: E704
def lor_t(a, b): return apply_broadcast2(a, b, 21)            # noqa: E704
def lxor_t(a, b): return apply_broadcast2(a, b, 22)           # noqa: E704
def lnand_t(a, b): return apply_broadcast2(a, b, 23)          # noqa: E704
def lnor_t(a, b): return apply_broadcast2(a, b, 24)           # noqa: E704
def lxnor_t(a, b): return apply_broadcast2(a, b, 25)          # noqa: E704
def landnot_t(a, b): return apply_broadcast2(a, b, 26)        # noqa: E704
def lnot_t(a): return _wrap(_raw(a) == 0)                     # noqa: E704
def elu_t(x): return apply_unary(x, 19)                       # noqa: E704
def selu_t(x): return apply_unary(x, 20)                      # noqa: E704
def silu_t(x): return apply_unary(x, 17)                      # noqa: E704
def gelu_t(x): return apply_unary(x, 18)                      # noqa: E704


def max_t(x):
    """Largest element as a Python scalar."""
    return _raw(x).max().item()


def min_t(x):
    return _raw(x).min().item()


reduce_max_f32, reduce_min_f32 = max_t, min_t


def sum1d_unrolled(m):
    return _raw(m).sum().item()


def variance(m, ddof=0, unbiased: bool = None, keepdims: bool = False):
    """``variance(m, ddof)`` over all elements as a float, or the reference's ``variance(x, axis, unbiased=True,
    keepdims=False)`` as a tensor (legacy/src/momijo/tensor/math.mojo:5156-5161): the second form is chosen by passing
    ``unbiased`` (or ``axis=None`` explicitly as ``ddof=None``)."""
    if unbiased is not None or ddof is None:
        r = _raw(m).double()
        ub = True if unbiased is None else bool(unbiased)
        from .tensor import _wrap
        return _wrap(r.var(unbiased=ub) if ddof is None else r.var(ddof, unbiased=ub, keepdim=keepdims))
    t = _raw(m).double().reshape(-1)
    n = t.numel()
    return float("nan") if n - ddof <= 0 else float(((t - t.mean()) ** 2).sum() / (n - ddof))


def std1d_unrolled(m, ddof: int = 0) -> float:
    v = variance(m, ddof)
    return math.sqrt(v) if v == v else v


def mean_axes_f64(x, axes, keepdims: bool = False):
    return _wrap(_raw(x).double().mean(dim=list(axes), keepdim=keepdims))


def normalize_(x, axis=None, eps: float = 1e-12) -> None:
    """In-place L2 normalisation along ``axis`` (whole tensor when None)."""
    t = _raw(x)
    f = t.double()
    n = f.pow(2).sum().sqrt() if axis is None else f.pow(2).sum(dim=axis, keepdim=True).sqrt()
    t.copy_((f / n.clamp_min(eps)).to(t.dtype))


def new_tensor_from_list(data, shape, from_f64=None):
    vals = [from_f64(float(v)) for v in data] if from_f64 is not None else list(data)
    return _wrap(torch.tensor(vals).reshape(list(shape)))


def one_hot_core_indices(indices, depth: int):
    """[N] integer indices -> [N, depth] float64 one-hot rows (out-of-range indices give a zero row)."""
    idx = _raw(indices).long().reshape(-1)
    out = torch.zeros(idx.numel(), depth, dtype=torch.float64)
    ok = (idx >= 0) & (idx < depth)
    out[torch.arange(idx.numel())[ok], idx[ok]] = 1.0
    return _wrap(out)


def _scatter_add(x, dim: int, index, src):
    t = _raw(x).clone()
    return _wrap(t.scatter_add_(dim, _raw(index).long(), _raw(src).to(t.dtype)))


for _d in (0, 1, 2, 3, 4):
    for _sfx in ("f32", "f64", "int"):
        globals()[f"scatter_add_dim{_d}_{_sfx}"] = (lambda d: (lambda x, index, src: _scatter_add(x, d, index, src)))(_d)


def f_vec(x):
    """Test function of the Jacobian helpers: [x0^2 + x1, sin(x0) * x1] for a 2-vector."""
    t = _raw(x).double()
    return _wrap(torch.stack([t[0] * t[0] + t[1], torch.sin(t[0]) * t[1]]))


def analytic_jacobian(x):
    t = _raw(x).double()
    return _wrap(torch.stack([torch.stack([2 * t[0], torch.ones_like(t[0])]),
                              torch.stack([torch.cos(t[0]) * t[1], torch.sin(t[0])])]))


def numeric_jacobian(fn, x, eps: float = 1e-6):
    """Central differences of ``fn`` (tensor -> tensor) at ``x``: [outputs, inputs]."""
    t = _raw(x).double().reshape(-1)
    cols = []
    for i in range(t.numel()):
        e = torch.zeros_like(t)
        e[i] = eps
        cols.append((_raw(fn(_wrap(t + e))).double().reshape(-1) - _raw(fn(_wrap(t - e))).double().reshape(-1)) / (2 * eps))
    return _wrap(torch.stack(cols, 1))


def safe_sqrt(x, eps: float = 1e-12):
    """Scalar form: ``sqrt(max(x, 0) + eps)`` (legacy/src/momijo/tensor/math.mojo:123-128). A tensor argument goes to
    the element-wise form of ``nanops``."""
    if isinstance(x, torch.Tensor):
        from .nanops import safe_sqrt as _tensor_form
        return _tensor_form(x, eps)
    return math.sqrt(max(float(x), 0.0) + eps)
