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


class OptParam:
    """Scalar parameter with its gradient (legacy/src/momijo/learn/optim/rmsprop.mojo:95-101)."""

    def __init__(self, value: float, grad: float = 0.0):
        self.value, self.grad = value, grad


def step_conv2d(opt: RMSprop, layer, dW, db):
    """RMSprop update of a ``Conv2d`` layer's weight and bias from explicit gradients
    (legacy/src/momijo/learn/optim/rmsprop.mojo:48-54)."""
    return opt.step_conv2d(layer, dW, db)
