"""Tape-style autograd names over ``torch.autograd``
(legacy/src/momijo/tensor/autograd.mojo:214-2213).

The reference keeps a struct-of-lists tape, supports Float32 only and walks a LIFO stack without
topological ordering, so a node reachable by two paths is processed twice. Here ``GradContext``
and ``GradTensor`` are thin handles over torch's engine (each node visited once) that keep the
reference's calling convention: every op takes the context first, ``requires_grad`` propagates
as ``a or b`` gated by ``no_grad_begin/no_grad_end``, and the tape losses ``nll_loss``,
``cross_entropy``, ``bce_with_logits`` and ``binary_cross_entropy`` keep their signatures.
"""
from __future__ import annotations

import torch
import torch.nn.functional as tF

from .tensor import Tensor, _raw, _wrap


class GradContext:
    def __init__(self):
        self.no_grad_depth = 0
        self.nodes = []

    def grad_enabled(self) -> bool:
        return self.no_grad_depth == 0

    def _track(self, value: torch.Tensor, requires_grad: bool) -> "GradTensor":
        gt = GradTensor(len(self.nodes), requires_grad, value)
        self.nodes.append(gt)
        return gt


def no_grad_begin(ctx: GradContext):
    ctx.no_grad_depth += 1


def no_grad_end(ctx: GradContext):
    ctx.no_grad_depth = max(0, ctx.no_grad_depth - 1)


def stop_gradient(ctx: GradContext, x: "GradTensor") -> "GradTensor":
    return ctx._track(x._val.detach(), False)


def _v(x):
    return x._val if isinstance(x, GradTensor) else (_raw(x) if isinstance(x, torch.Tensor) else x)


def _rg(*xs):
    return any(isinstance(x, GradTensor) and x.requires_grad for x in xs)


class GradTensor:
    """``(id, requires_grad)`` handle; the value lives on the context's tape."""

    def __init__(self, id: int, requires_grad: bool, value: torch.Tensor):
        self.id, self.requires_grad, self._val = id, requires_grad, value

    @staticmethod
    def from_tensor(ctx: GradContext, t, requires_grad: bool = False) -> "GradTensor":
        v = _raw(t).detach().clone().float()
        rg = requires_grad and ctx.grad_enabled()
        if rg:
            v.requires_grad_(True)
        return ctx._track(v, rg)

    def tensor(self, ctx: GradContext = None):
        return _wrap(self._val.detach())

    def grad(self, ctx: GradContext = None):
        g = self._val.grad
        return _wrap(g if g is not None else torch.zeros_like(self._val))

    # ---- read-only accessors (legacy/src/momijo/tensor/autograd.mojo:320-365, 1079-1105) -------------------
    @staticmethod
    def from_randn(ctx: GradContext, shape, requires_grad: bool = False) -> "GradTensor":
        return GradTensor.from_tensor(ctx, torch.randn(list(shape)), requires_grad)

    @staticmethod
    def has_matmul2d() -> bool:
        return True

    def value(self, ctx: GradContext = None):
        return _wrap(self._val.detach().clone())

    def shape(self, ctx: GradContext = None):
        return list(self._val.shape)

    def numel(self, ctx: GradContext = None) -> int:
        return self._val.numel()

    def item(self, ctx: GradContext = None) -> float:
        return float(self._val.detach().reshape(-1)[0])

    def at_flat(self, ctx: GradContext, i: int) -> float:
        return float(self._val.detach().reshape(-1)[i])

    def to_list(self, ctx: GradContext = None):
        return self._val.detach().reshape(-1).tolist()

    def to_string(self, ctx: GradContext = None) -> str:
        return str(_wrap(self._val.detach()))

    def to_Float32(self, ctx: GradContext = None) -> "GradTensor":
        return self

    def to_int_value(self, ctx: GradContext = None):
        return _wrap(self._val.detach().to(torch.int64))

    def to_float32_value(self, ctx: GradContext = None):
        return _wrap(self._val.detach().to(torch.float32))

    def _cmp_scalar(self, ctx, fn, s):
        """Comparison masks are 0/1 floats on a fresh untracked node (autograd.mojo:1291-1340)."""
        return ctx._track(fn(self._val.detach(), s).to(torch.float32), False)

    def eq_scalar(self, ctx, s): return self._cmp_scalar(ctx, torch.eq, s)
    def ne_scalar(self, ctx, s): return self._cmp_scalar(ctx, torch.ne, s)
    def lt_scalar(self, ctx, s): return self._cmp_scalar(ctx, torch.lt, s)
    def le_scalar(self, ctx, s): return self._cmp_scalar(ctx, torch.le, s)
    def gt_scalar(self, ctx, s): return self._cmp_scalar(ctx, torch.gt, s)
    def ge_scalar(self, ctx, s): return self._cmp_scalar(ctx, torch.ge, s)

    def sum_axis(self, ctx, axis: int, keepdims: bool = False): return self.sum(ctx, axis, keepdims)
    def mean_axis(self, ctx, axis: int, keepdims: bool = False): return self.mean(ctx, axis, keepdims)

    def select(self, ctx, mask, other):
        """``where(mask, self, other)`` (autograd.mojo:816-817)."""
        m = _raw(mask).bool() if isinstance(mask, torch.Tensor) else torch.as_tensor(mask).bool()
        return self._op(ctx, lambda a, b: torch.where(m, a, b), other)

    def backward(self, ctx: GradContext = None, grad=None):
        """Seeds ones (like the reference) and back-propagates once through every node."""
        seed = torch.ones_like(self._val) if grad is None else _raw(grad)
        for n in (ctx.nodes if ctx is not None else []):
            if n._val.is_leaf and n._val.grad is not None:
                n._val.grad = None
        self._val.backward(seed)

    def _op(self, ctx, fn, *others):
        rg = _rg(self, *others) and ctx.grad_enabled()
        if rg:
            out = fn(self._val, *[_v(o) for o in others])
        else:
            with torch.no_grad():
                out = fn(self._val, *[_v(o) for o in others])
        return ctx._track(out, rg)

    # binary (tensor / GradTensor / scalar operands)
    def add(self, ctx, o): return self._op(ctx, lambda a, b: a + b, o)
    def sub(self, ctx, o): return self._op(ctx, lambda a, b: a - b, o)
    def mul(self, ctx, o): return self._op(ctx, lambda a, b: a * b, o)
    def div(self, ctx, o): return self._op(ctx, lambda a, b: a / b, o)
    add_scalar = add
    sub_scalar = sub
    mul_scalar = mul
    div_scalar = div

    def maximum_scalar(self, ctx, c): return self._op(ctx, lambda a: torch.clamp(a, min=c))
    def minimum_scalar(self, ctx, c): return self._op(ctx, lambda a: torch.clamp(a, max=c))
    def pow_scalar(self, ctx, p): return self._op(ctx, lambda a: a ** p)

    # unary
    def neg(self, ctx): return self._op(ctx, torch.neg)
    def square(self, ctx): return self._op(ctx, torch.square)
    def sqrt(self, ctx): return self._op(ctx, torch.sqrt)
    def exp(self, ctx): return self._op(ctx, torch.exp)
    def log(self, ctx): return self._op(ctx, torch.log)
    def tanh(self, ctx): return self._op(ctx, torch.tanh)
    def sigmoid(self, ctx): return self._op(ctx, torch.sigmoid)
    def relu(self, ctx): return self._op(ctx, torch.relu)
    def leaky_relu(self, ctx, slope=0.01): return self._op(ctx, lambda a: tF.leaky_relu(a, slope))
    def abs(self, ctx): return self._op(ctx, torch.abs)
    def sign(self, ctx): return self._op(ctx, torch.sign)
    def floor(self, ctx): return self._op(ctx, torch.floor)
    def ceil(self, ctx): return self._op(ctx, torch.ceil)
    def round(self, ctx): return self._op(ctx, torch.round)
    def log1p(self, ctx): return self._op(ctx, torch.log1p)
    def expm1(self, ctx): return self._op(ctx, torch.expm1)

    # reductions
    def sum_all(self, ctx): return self._op(ctx, torch.sum)
    def mean_all(self, ctx): return self._op(ctx, torch.mean)
    def sum(self, ctx, axis=None, keepdims=False):
        return self._op(ctx, (lambda a: a.sum()) if axis is None else (lambda a: a.sum(axis, keepdim=keepdims)))

    def mean(self, ctx, axis=None, keepdims=False):
        return self._op(ctx, (lambda a: a.mean()) if axis is None else (lambda a: a.mean(axis, keepdim=keepdims)))

    def std(self, ctx, axis=None, keepdims=False, eps=0.0):
        """Biased, with eps inside the sqrt (autograd.mojo:181, 1877-1916)."""
        def f(a):
            v = a.var(unbiased=False) if axis is None else a.var(axis, unbiased=False, keepdim=keepdims)
            return torch.sqrt(v + eps)
        return self._op(ctx, f)

    # shapes
    def reshape(self, ctx, shape): return self._op(ctx, lambda a: a.reshape(list(shape)))
    def permute(self, ctx, axes): return self._op(ctx, lambda a: a.permute(list(axes)))
    def flatten(self, ctx): return self._op(ctx, lambda a: a.reshape(-1))
    def transpose2d(self, ctx): return self._op(ctx, lambda a: a.t())
    def squeeze(self, ctx, axis=None): return self._op(ctx, lambda a: a.squeeze() if axis is None else a.squeeze(axis))
    def unsqueeze(self, ctx, axis): return self._op(ctx, lambda a: a.unsqueeze(axis))
    def repeat(self, ctx, reps): return self._op(ctx, lambda a: a.repeat(*reps))

    # indexing
    def gather(self, ctx, axis, index): return self._op(ctx, lambda a: torch.gather(a, axis, _v(index).long()))
    def index_axis(self, ctx, axis, i): return self._op(ctx, lambda a: a.select(axis, i))
    def take(self, ctx, index): return self._op(ctx, lambda a: torch.take(a, _v(index).long()))
    def scatter(self, ctx, axis, index, src): return self._op(ctx, lambda a, s: a.scatter(axis, _v(index).long(), s), src)
    def masked_select(self, ctx, mask): return self._op(ctx, lambda a: torch.masked_select(a, _v(mask) != 0))
    def where(self, ctx, cond, other): return self._op(ctx, lambda a, b: torch.where(_v(cond) != 0, a, b), other)

    # products
    def matmul2d(self, ctx, o): return self._op(ctx, lambda a, b: a @ b, o)
    matmul = matmul2d
    def tensordot(self, ctx, o, axes=1): return self._op(ctx, lambda a, b: torch.tensordot(a, b, dims=axes), o)

    # composed
    def softmax(self, ctx, axis=-1): return self._op(ctx, lambda a: torch.softmax(a, axis))
    def logsumexp(self, ctx, axis=-1, keepdims=False): return self._op(ctx, lambda a: torch.logsumexp(a, axis, keepdim=keepdims))
    def log_softmax(self, ctx, axis=-1): return self._op(ctx, lambda a: torch.log_softmax(a, axis))

    def clip(self, ctx, lo, hi):
        """Gradient is routed to ``lo`` / ``hi`` when they are tape nodes (autograd.mojo:1969-1998)."""
        return self._op(ctx, lambda a, l, h: torch.minimum(torch.maximum(a, torch.as_tensor(l, dtype=a.dtype)),
                                                           torch.as_tensor(h, dtype=a.dtype)), lo, hi)

    clamp = clip

    # comparisons (no gradient)
    def eq(self, ctx, o): return ctx._track((self._val == _v(o)).float(), False)
    def ne(self, ctx, o): return ctx._track((self._val != _v(o)).float(), False)
    def lt(self, ctx, o): return ctx._track((self._val < _v(o)).float(), False)
    def le(self, ctx, o): return ctx._track((self._val <= _v(o)).float(), False)
    def gt(self, ctx, o): return ctx._track((self._val > _v(o)).float(), False)
    def ge(self, ctx, o): return ctx._track((self._val >= _v(o)).float(), False)


def _reduce(x, reduction):
    return x.mean() if reduction == "mean" else (x.sum() if reduction == "sum" else x)


def nll_loss(ctx, log_probs: GradTensor, target, axis: int = 1, class_weight=None, reduction="mean"):
    t = _v(target).long()
    w = _v(class_weight) if class_weight is not None else None

    def f(lp):
        picked = -torch.gather(lp, axis, t.unsqueeze(axis)).squeeze(axis)
        if w is not None:
            ww = w[t]
            picked = picked * ww
            if reduction == "mean":
                return picked.sum() / ww.sum()
        return _reduce(picked, reduction)
    return log_probs._op(ctx, f)


def cross_entropy(ctx, logits: GradTensor, target, axis: int = 1, class_weight=None, reduction="mean"):
    return nll_loss(ctx, logits.log_softmax(ctx, axis), target, axis, class_weight, reduction)


def bce_with_logits(ctx, logits: GradTensor, target, pos_weight=None, reduction="mean"):
    t = _v(target).float()
    pw = _v(pos_weight) if pos_weight is not None else None

    def f(x):
        loss = x.clamp_min(0) - x * t + torch.log1p(torch.exp(-x.abs()))
        if pw is not None:
            loss = loss * (1 + (pw - 1) * t)
        return _reduce(loss, reduction)
    return logits._op(ctx, f)


def binary_cross_entropy(ctx, probs: GradTensor, target, eps=1e-12, weight=None, reduction="mean"):
    t = _v(target).float()
    w = _v(weight) if weight is not None else None

    def f(p):
        p = p.clamp(eps, 1 - eps)
        loss = -(t * p.log() + (1 - t) * (1 - p).log())
        if w is not None:
            loss = loss * w
        return _reduce(loss, reduction)
    return probs._op(ctx, f)


# ---- op tags, the struct-of-lists tape record and small helpers of the reference
# (legacy/src/momijo/tensor/autograd.mojo:18-300, 2179-2200). Differentiation itself runs on torch autograd
# (``GradTensor`` above); ``Tape`` keeps the reference's bookkeeping layout for code that inspects or builds
# tapes directly, and the tag functions return the same numbers.
_TAGS = {
    "LEAF": 0, "ADD": 1, "MUL": 2, "ADDS": 3, "MULS": 4, "SUM_ALL": 5, "MEAN_ALL": 6, "RESHAPE": 7, "PERMUTE": 8,
    "SUM_AX": 9, "MEAN_AX": 10, "NEG": 11, "SUB": 12, "DIVS": 13, "SQUARE": 14, "POWS": 15, "TRANSPOSE2D": 16,
    "FLATTEN": 17, "MATMUL2D": 18, "MAXS": 19, "MINS": 20, "RELU": 21, "LRELU": 22, "REPEAT": 23, "GATHER": 24,
    "INDEX_AXIS": 25, "TAKE": 26, "SCATTER": 27, "MASKED_SELECT": 28, "MASKED_SELECT_ELEM": 29, "DIV": 30,
    "CLIP": 31, "CLAMP_DISABLED": 32, "CLAMP_DISA": 31, "TENSORDOT": 51, "SQRT": 60, "EXP": 61, "LOG": 62,
    "TANH": 63, "SIGMOID": 64, "ABS": 65, "SIGN": 66, "FLOOR": 67, "CEIL": 68, "ROUND": 69, "LOG1P": 70,
    "EXPM1": 71, "CLAMP": 72, "STD": 80, "WHERE": 90,
}
for _tag_name, _tag_id in _TAGS.items():
    globals()[f"TAG_{_tag_name}"] = (lambda v: (lambda: v))(_tag_id)


class Tape:
    """values / grads / op_tags / parents / scalars / shapes / orders / axes / keep, one entry per node."""

    def __init__(self):
        self.values, self.grads, self.op_tags, self.parents = [], [], [], []
        self.scalars, self.shapes, self.orders, self.axes, self.keep = [], [], [], [], []

    def _push_common(self, val, op: int, p0: int = -1, p1: int = -1, s: float = 0.0, shp=(), ord=(), ax: int = -1,
                     kd: bool = False) -> int:
        v = _v(val)
        self.values.append(v.clone())
        self.grads.append(torch.zeros_like(v))
        self.op_tags.append(op)
        self.parents.append([p0, p1])
        self.scalars.append(s)
        self.shapes.append(list(shp))
        self.orders.append(list(ord))
        self.axes.append(ax)
        self.keep.append(kd)
        return len(self.values) - 1

    def add_leaf(self, x) -> int:
        return self._push_common(x, 0)

    def add_node(self, val, op: int, p0: int = -1, p1: int = -1, **kw) -> int:
        return self._push_common(val, op, p0, p1, **kw)

    def add_unary(self, val, op: int, p: int, s: float = 0.0, shp=(), ord=(), ax: int = -1, kd: bool = False) -> int:
        return self._push_common(val, op, p, -1, s, shp, ord, ax, kd)

    def add_binary(self, val, op: int, p0: int, p1: int) -> int:
        return self._push_common(val, op, p0, p1)

    def __len__(self):
        return len(self.values)

    def zero_grads(self):
        for g in self.grads:
            g.zero_()


def needs_grad(flag_a: bool, flag_b: bool = False) -> bool:
    return bool(flag_a or flag_b)


def shape_like(x):
    return list(_v(x).shape)


def broadcast_to_shape(x, shape):
    from .tensor import _wrap
    t = _v(x)
    return _wrap(t.clone() if list(t.shape) == list(shape) else t.expand(list(shape)).clone())


def no_grad_do(ctx: GradContext, f) -> None:
    """Run ``f()`` with gradient tracking off, restoring it afterwards even if ``f`` raises."""
    no_grad_begin(ctx)
    try:
        f()
    finally:
        no_grad_end(ctx)


def _mask_out(t):
    from .tensor import _wrap
    return _wrap(t.to(torch.int64))


def mask_not(mask): return _mask_out(_v(mask) == 0)                                   # noqa: E704
def mask_and(a, b): return _mask_out((_v(a) != 0) & (_v(b) != 0))                     # noqa: E704
def mask_or(a, b): return _mask_out((_v(a) != 0) | (_v(b) != 0))                      # noqa: E704


def where(ctx: GradContext, mask, a: "GradTensor", b: "GradTensor") -> "GradTensor":
    """``mask != 0 ? a : b`` with gradients to both branches (legacy/src/momijo/tensor/autograd.mojo:2159-2180)."""
    return a.where(ctx, mask, b)
