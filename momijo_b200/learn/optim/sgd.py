"""``SGD(lr=0.01)``: ``w <- w - lr * g`` (legacy/src/momijo/learn/optim/sgd.mojo:14-53).
``momentum``, ``weight_decay`` and ``nesterov`` are extensions that default to off."""
import torch

from .base import _PerLayerOptimizer


class SGD(_PerLayerOptimizer):
    def __init__(self, params=None, lr=0.01, momentum=0.0, weight_decay=0.0, nesterov=False):
        if isinstance(params, (int, float)):  # SGD(0.1): reference positional lr
            params, lr = None, float(params)
        super().__init__(params, lr)
        self.momentum, self.weight_decay, self.nesterov = momentum, weight_decay, nesterov

    def _update(self, key, p, g):
        g = g.to(p.dtype)
        if self.weight_decay:
            g = g + self.weight_decay * p
        if self.momentum:
            buf = self.state.get(key)
            if buf is None or buf.shape != g.shape:
                buf = g.clone()
            else:
                buf.mul_(self.momentum).add_(g)
            self.state[key] = buf
            g = g + self.momentum * buf if self.nesterov else buf
        p.sub_(self.lr * g)
