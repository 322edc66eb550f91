"""Activation functions for scalars, lists and tensors
(legacy/src/momijo/learn/nn/activations.mojo:104-667)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tF


def _t(x):
    if isinstance(x, torch.Tensor):
        return x, "t"
    if isinstance(x, (list, tuple)):
        return torch.tensor(x, dtype=torch.float64), "l"
    return torch.tensor(float(x), dtype=torch.float64), "s"


def _back(y, kind):
    if kind == "t":
        return y
    if kind == "l":
        return y.tolist()
    return float(y)


def _wrap(fn):
    def f(x, *a, **k):
        t, kind = _t(x)
        return _back(fn(t, *a, **k), kind)
    f.__name__ = fn.__name__
    f.__doc__ = fn.__doc__
    return f


@_wrap
def relu(x):
    return torch.relu(x)


@_wrap
def leaky_relu(x, slope=0.01):
    return tF.leaky_relu(x, slope)


@_wrap
def relu6(x):
    return torch.clamp(x, 0.0, 6.0)


@_wrap
def sigmoid(x):
    return torch.sigmoid(x)


@_wrap
def tanh(x):
    return torch.tanh(x)


@_wrap
def silu(x):
    return tF.silu(x)


@_wrap
def gelu(x):
    """tanh approximation, as in the reference."""
    return tF.gelu(x, approximate="tanh")


@_wrap
def elu(x, alpha=1.0):
    return tF.elu(x, alpha)


@_wrap
def selu(x):
    return tF.selu(x)


@_wrap
def hard_sigmoid(x):
    return torch.clamp(0.2 * x + 0.5, 0.0, 1.0)


@_wrap
def hard_swish(x):
    return x * torch.clamp(x + 3.0, 0.0, 6.0) / 6.0


@_wrap
def softplus(x, beta=1.0, threshold=20.0):
    return tF.softplus(x, beta, threshold)


@_wrap
def softsign(x):
    return x / (1.0 + x.abs())


@_wrap
def softshrink(x, lambd=0.5):
    return tF.softshrink(x, lambd)


@_wrap
def hardshrink(x, lambd=0.5):
    return tF.hardshrink(x, lambd)


@_wrap
def mish(x):
    return x * torch.tanh(tF.softplus(x))


@_wrap
def threshold(x, thr=0.0, value=0.0):
    return torch.where(x > thr, x, torch.full_like(x, value))


@_wrap
def hardtanh(x, lo=-1.0, hi=1.0):
    return torch.clamp(x, lo, hi)


def softmax_stable(x, axis=-1):
    t, kind = _t(x)
    return _back(torch.softmax(t, dim=axis), kind)


softmax = softmax_stable


def log_softmax(x, axis=-1):
    """Exact log-softmax (the reference's free function uses a soft row-max approximation,
    legacy/src/momijo/tensor/math.mojo:463-478)."""
    t, kind = _t(x)
    return _back(torch.log_softmax(t, dim=axis), kind)


# the reference spells these two both ways (legacy/src/momijo/learn/nn/activations.mojo:533-560)
hardsigmoid = hard_sigmoid
swish = silu
