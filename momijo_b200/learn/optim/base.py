"""Shared plumbing of the per-layer optimizers.

The reference optimizers are driven per layer: ``opt.step_linear(layer, dW, db)`` /
``opt.step_conv2d(layer, dW, db)`` with one state object per optimizer instance, i.e. one
optimizer per layer (legacy/src/momijo/learn/optim/adamw.mojo:39-147). The same objects also
accept ``params`` and then offer ``step()`` / ``zero_grad()`` over ``.grad`` like the generic
RMSprop of the reference (rmsprop.mojo:107-333).
"""
from __future__ import annotations

import torch


class _PerLayerOptimizer:
    def __init__(self, params=None, lr=1e-3):
        self.lr = lr
        self.params = list(params) if params is not None else []
        self.state = {}

    # --- update rule, implemented by subclasses: returns nothing, updates p in place ---
    def _update(self, key, p: torch.Tensor, g: torch.Tensor):
        raise NotImplementedError

    @torch.no_grad()
    def step_linear(self, layer, dW, db=None):
        self._update("W", layer.weight, dW)
        if db is not None and layer.bias_t.numel():
            self._update("B", layer.bias_t, db)

    step_conv2d = step_linear

    @torch.no_grad()
    def step_tensor(self, p, g, key=None):
        self._update(key if key is not None else id(p), p, g)

    @torch.no_grad()
    def step(self):
        for i, p in enumerate(self.params):
            if p.grad is not None:
                self._update(("p", i), p, p.grad)

    def zero_grad(self, set_to_none: bool = True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def get_lr(self):
        return self.lr

    def set_lr(self, lr):
        self.lr = lr

    @property
    def param_groups(self):
        return [{"lr": self.lr, "params": self.params}]
