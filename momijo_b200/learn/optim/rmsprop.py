"""``RMSprop(lr=1e-3, alpha=.99, eps=1e-8, weight_decay, momentum, centered, decoupled)``:
eps inside the sqrt, momentum buffer, centered variant, decoupled decay after the step
(legacy/src/momijo/learn/optim/rmsprop.mojo:239-331)."""
import torch

from .base import _PerLayerOptimizer


class RMSprop(_PerLayerOptimizer):
    def __init__(self, params=None, lr=1e-3, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0,
                 centered=False, decoupled=False):
        if isinstance(params, (int, float)):
            params, lr = None, float(params)
        super().__init__(params, lr)
        self.alpha, self.eps, self.weight_decay = alpha, eps, weight_decay
        self.momentum, self.centered, self.decoupled = momentum, centered, decoupled

    def _update(self, key, p, g):
        g = g.to(p.dtype)
        st = self.state.get(key)
        if st is None or st["sq"].shape != g.shape:
            st = {"sq": torch.zeros_like(p), "mg": torch.zeros_like(p), "buf": torch.zeros_like(p)}
            self.state[key] = st
        if self.weight_decay and not self.decoupled:
            g = g + self.weight_decay * p
        st["sq"].mul_(self.alpha).addcmul_(g, g, value=1 - self.alpha)
        avg = st["sq"]
        if self.centered:
            st["mg"].mul_(self.alpha).add_(g, alpha=1 - self.alpha)
            avg = avg - st["mg"] ** 2
        denom = (avg + self.eps).sqrt()
        if self.momentum:
            st["buf"].mul_(self.momentum).add_(g / denom)
            p.sub_(self.lr * st["buf"])
        else:
            p.sub_(self.lr * g / denom)
        if self.weight_decay and self.decoupled:
            p.mul_(1 - self.lr * self.weight_decay)


def _rms_set_params(self, ps) -> None:
    """Scalar mode: a list of ``OptParam`` (value, grad) pairs with fresh state (rmsprop.mojo:165-183)."""
    self._scalars, self._tensor_pair = list(ps), None
    self.params = []
    self.state = {}


def _rms_set_params_tensor(self, params, grads) -> None:
    """Tensor mode: one parameter tensor and the gradient tensor the caller fills before each ``step``
    (rmsprop.mojo:185-204)."""
    if tuple(params.shape) != tuple(grads.shape):
        raise ValueError("RMSprop.set_params_tensor: parameter and gradient shapes differ")
    self._scalars, self._tensor_pair = None, (params, grads)
    self.params = []
    self.state = {}


def _rms_step(self):
    pair, scalars = getattr(self, "_tensor_pair", None), getattr(self, "_scalars", None)
    with torch.no_grad():
        if pair is not None:
            self._update("tensor", pair[0], pair[1])
        elif scalars is not None:
            for i, sp in enumerate(scalars):
                t = torch.tensor([float(sp.value)], dtype=torch.float64)
                self._update(("s", i), t, torch.tensor([float(sp.grad)], dtype=torch.float64))
                sp.value = float(t[0])
        else:
            _PerLayerOptimizer.step(self)


def _rms_zero_grad(self, set_to_none: bool = True):
    pair, scalars = getattr(self, "_tensor_pair", None), getattr(self, "_scalars", None)
    if pair is not None:
        pair[1].zero_()
    elif scalars is not None:
        for sp in scalars:
            sp.grad = 0.0
    else:
        _PerLayerOptimizer.zero_grad(self, set_to_none)


RMSprop.set_params, RMSprop.set_params_tensor = _rms_set_params, _rms_set_params_tensor
RMSprop.step, RMSprop.zero_grad = _rms_step, _rms_zero_grad


class OptParam:
    """Scalar parameter with its gradient (legacy/src/momijo/learn/optim/rmsprop.mojo:95-101)."""

    def __init__(self, value: float, grad: float = 0.0):
        self.value, self.grad = value, grad


def step_conv2d(opt: RMSprop, layer, dW, db):
    """RMSprop update of a ``Conv2d`` layer's weight and bias from explicit gradients
    (legacy/src/momijo/learn/optim/rmsprop.mojo:48-54)."""
    return opt.step_conv2d(layer, dW, db)
