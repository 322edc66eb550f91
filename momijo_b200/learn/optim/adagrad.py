"""``Adagrad(lr, eps, weight_decay)``: ``g += wd*w; acc += g^2; w -= lr*g/(sqrt(acc)+eps)``
(legacy/src/momijo/learn/optim/adagrad.mojo:59-83)."""
import torch

from .base import _PerLayerOptimizer


class Adagrad(_PerLayerOptimizer):
    def __init__(self, params=None, lr=1e-2, eps=1e-10, weight_decay=0.0):
        if isinstance(params, (int, float)):
            params, lr = None, float(params)
        super().__init__(params, lr)
        self.eps, self.weight_decay = eps, weight_decay

    def _update(self, key, p, g):
        g = g.to(p.dtype)
        if self.weight_decay:
            g = g + self.weight_decay * p
        acc = self.state.get(key)
        if acc is None or acc.shape != g.shape:
            acc = torch.zeros_like(p)
            self.state[key] = acc
        acc.addcmul_(g, g)
        p.sub_(self.lr * g / (acc.sqrt() + self.eps))


def adagrad_update_scalar(param: float, grad: float, acc: float, lr: float, eps: float, weight_decay: float):
    """One Adagrad step on a scalar: returns (new parameter, new accumulator)
    (legacy/src/momijo/learn/optim/adagrad.mojo:59-77)."""
    import math
    g = grad + weight_decay * param if weight_decay != 0.0 else grad
    acc_new = acc + g * g
    denom = math.sqrt(acc_new) + eps
    if denom <= 0.0:
        denom = eps
    return param - lr * g / denom, acc_new
