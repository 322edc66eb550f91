"""Math functions (legacy/src/momijo/tensor/math.mojo): elementwise/unary/compare/logical ops,
reductions, ``softmax`` (last axis, max-subtracted) and exact ``log_softmax``, ``lerp/dot/
normalize``, ``Complex128`` helpers, ``scatter_add``, and the small linear algebra set
(``qr/inv/svd/cholesky/solve/matmul2d``)."""
from __future__ import annotations

import torch

from .errors import ErrorKind, TensorError, check_matmul, raise_or
from .tensor import Tensor, _mask, _raw, _wrap


def _t(x):
    return _raw(x) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _u(fn):
    def f(x, *a, **k):
        return _wrap(fn(_t(x), *a, **k))
    return f


exp_t, log_t, sqrt_t, abs_t, neg_t = _u(torch.exp), _u(torch.log), _u(torch.sqrt), _u(torch.abs), _u(torch.neg)
sin_t, cos_t, tan_t, tanh_t, sigmoid_t = _u(torch.sin), _u(torch.cos), _u(torch.tan), _u(torch.tanh), _u(torch.sigmoid)
floor_t, ceil_t, round_t, sign_t = _u(torch.floor), _u(torch.ceil), _u(torch.round), _u(torch.sign)
log1p_t, expm1_t, square_t, relu_t = _u(torch.log1p), _u(torch.expm1), _u(torch.square), _u(torch.relu)


def add_t(a, b): return _wrap(_t(a) + _t(b))
def sub_t(a, b): return _wrap(_t(a) - _t(b))
def mul_t(a, b): return _wrap(_t(a) * _t(b))


def div_t(a, b):
    a, b = _t(a), _t(b)
    if not a.dtype.is_floating_point and not b.dtype.is_floating_point:
        a, b = a.double(), b.double()
    return _wrap(a / b)


def pow_t(a, b): return _wrap(torch.pow(_t(a), _t(b) if isinstance(b, torch.Tensor) else b))
def maximum_t(a, b): return _wrap(torch.maximum(_t(a), _t(b)))
def minimum_t(a, b): return _wrap(torch.minimum(_t(a), _t(b)))


def and_t(a, b): return _wrap((_mask(_t(a)) & _mask(_t(b))).to(torch.int64))
def or_t(a, b): return _wrap((_mask(_t(a)) | _mask(_t(b))).to(torch.int64))
def xor_t(a, b): return _wrap((_mask(_t(a)) ^ _mask(_t(b))).to(torch.int64))
def not_t(a): return _wrap((~_mask(_t(a))).to(torch.int64))


def eq_t(a, b): return _wrap((_t(a) == _t(b)).to(torch.int64))
def ne_t(a, b): return _wrap((_t(a) != _t(b)).to(torch.int64))
def lt_t(a, b): return _wrap((_t(a) < _t(b)).to(torch.int64))
def le_t(a, b): return _wrap((_t(a) <= _t(b)).to(torch.int64))
def gt_t(a, b): return _wrap((_t(a) > _t(b)).to(torch.int64))
def ge_t(a, b): return _wrap((_t(a) >= _t(b)).to(torch.int64))


def reciprocal(x): return _wrap(1.0 / _t(x).double() if not _t(x).dtype.is_floating_point else 1.0 / _t(x))
def reciprocal_scalar(s): return 1.0 / s


def safe_div(a, b, fill=0.0):
    a, b = _t(a).double(), _t(b).double()
    return _wrap(torch.where(b != 0, a / torch.where(b != 0, b, torch.ones_like(b)), torch.full_like(a, fill)))


def safe_div_scalar(a, s, fill=0.0):
    return _wrap(_t(a).double() / s) if s != 0 else _wrap(torch.full_like(_t(a).double(), fill))


def softmax(x, axis: int = -1):
    return _wrap(torch.softmax(_t(x).float() if not _t(x).dtype.is_floating_point else _t(x), dim=axis))


def log_softmax(x, axis: int = -1):
    return _wrap(torch.log_softmax(_t(x).float() if not _t(x).dtype.is_floating_point else _t(x), dim=axis))


def logsumexp(x, axis: int = -1, keepdims=False):
    return _wrap(torch.logsumexp(_t(x), dim=axis, keepdim=keepdims))


def sum(x, axis=None, keepdims=False):
    return _wrap(_t(x).sum() if axis is None else _t(x).sum(dim=axis, keepdim=keepdims))


def mean(x, axis=None, keepdims=False):
    r = _t(x)
    r = r.double() if not r.dtype.is_floating_point else r
    return _wrap(r.mean() if axis is None else r.mean(dim=axis, keepdim=keepdims))


def std(x, axis=None, keepdims=False, unbiased=False):
    r = _t(x)
    r = r.double() if not r.dtype.is_floating_point else r
    return _wrap(r.std(unbiased=unbiased) if axis is None else r.std(dim=axis, keepdim=keepdims, unbiased=unbiased))


def var(x, axis=None, keepdims=False, unbiased=False):
    r = _t(x)
    r = r.double() if not r.dtype.is_floating_point else r
    return _wrap(r.var(unbiased=unbiased) if axis is None else r.var(dim=axis, keepdim=keepdims, unbiased=unbiased))


def min(x, axis=None, keepdims=False):
    return _wrap(_t(x).min() if axis is None else _t(x).min(dim=axis, keepdim=keepdims).values)


def max(x, axis=None, keepdims=False):
    return _wrap(_t(x).max() if axis is None else _t(x).max(dim=axis, keepdim=keepdims).values)


def prod(x, axis=None, keepdims=False):
    return _wrap(_t(x).prod() if axis is None else _t(x).prod(dim=axis, keepdim=keepdims))


def argmax(x, axis=None):
    return _wrap(_t(x).argmax() if axis is None else _t(x).argmax(dim=axis))


def argmin(x, axis=None):
    return _wrap(_t(x).argmin() if axis is None else _t(x).argmin(dim=axis))


def lerp(a, b, w):
    return _wrap(_t(a) + (_t(b) - _t(a)) * w)


def dot(a, b):
    return _wrap(torch.dot(_t(a).reshape(-1), _t(b).reshape(-1)))


def normalize(x, axis: int = -1, eps: float = 1e-12):
    r = _t(x)
    return _wrap(r / r.norm(dim=axis, keepdim=True).clamp_min(eps))


def matmul2d(a, b):
    """2-D x 2-D; wrong shapes raise (the reference returns zeros, math.mojo:7858-7859; lenient
    mode keeps that)."""
    a, b = _t(a), _t(b)
    bad = a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]
    if bad:
        fb = raise_or(check_matmul(a.shape, b.shape) if a.dim() == 2 and b.dim() == 2 else
                      __import__("momijo_b200.tensor.errors", fromlist=["Status"]).Status.fail(ErrorKind.SHAPE, "matmul2d needs 2-D operands"),
                      torch.zeros(a.shape[0] if a.dim() else 0, b.shape[-1] if b.dim() else 0))
        return _wrap(fb)
    if not a.dtype.is_floating_point and not b.dtype.is_floating_point:
        a, b = a.float(), b.float()
    return _wrap(a @ b)


def qr(a):
    q, r = torch.linalg.qr(_t(a))
    return _wrap(q), _wrap(r)


def inv(a): return _wrap(torch.linalg.inv(_t(a)))
def cholesky(a): return _wrap(torch.linalg.cholesky(_t(a)))
def solve(a, b): return _wrap(torch.linalg.solve(_t(a), _t(b)))


def svd(a):
    u, s, vh = torch.linalg.svd(_t(a), full_matrices=False)
    return _wrap(u), _wrap(s), _wrap(vh)


def scatter_add(x, axis: int, index, src):
    return _wrap(_t(x).scatter_add(axis, _t(index).long(), _t(src)))


scatter_add_dim0 = lambda x, index, src: scatter_add(x, 0, index, src)  # noqa: E731
scatter_add_dim1 = lambda x, index, src: scatter_add(x, 1, index, src)  # noqa: E731


def jacobian(fn, x):
    return _wrap(torch.autograd.functional.jacobian(fn, _t(x)))


class Complex128:
    def __init__(self, re=0.0, im=0.0):
        self.re, self.im = float(re), float(im)

    def __add__(self, o): return Complex128(self.re + o.re, self.im + o.im)
    def __sub__(self, o): return Complex128(self.re - o.re, self.im - o.im)
    def __mul__(self, o): return Complex128(self.re * o.re - self.im * o.im, self.re * o.im + self.im * o.re)
    def abs(self): return (self.re ** 2 + self.im ** 2) ** 0.5
    def real(self): return self.re
    def imag(self): return self.im
    def conj(self): return Complex128(self.re, -self.im)
    def __repr__(self): return f"({self.re}+{self.im}j)"


def complex(re, im):
    return _wrap(torch.complex(_t(re).double(), _t(im).double()))


def complex_abs(z): return _wrap(_t(z).abs())
def complex_real(z): return _wrap(_t(z).real)
def complex_imag(z): return _wrap(_t(z).imag)


# scalar shims, op-id dispatchers, logical and in-place ops (see math_compat for the op-id tables)
from .math_compat import *  # noqa: F401,F403,E402
from .math_compat import (expm1_32, log1p32, pow32, abs32, sqrt32, exp32, log32, sin32, cos32, tan32, tanh32,  # noqa: F401,E402
                          floor32, ceil32, round32, sign32, sigmoid32, silu32, gelu32, elu32, selu32)
