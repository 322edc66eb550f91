"""``Adam`` with decoupled decay as the reference applies it
(legacy/src/momijo/learn/optim/adam.mojo:105-175); state is re-initialised when the gradient
size changes."""
import torch

from .base import _PerLayerOptimizer


class Adam(_PerLayerOptimizer):
    def __init__(self, params=None, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
                 betas=None):
        if isinstance(params, (int, float)):
            params, lr = None, float(params)
        super().__init__(params, lr)
        if betas is not None:
            beta1, beta2 = betas
        self.beta1, self.beta2, self.eps, self.weight_decay = beta1, beta2, eps, weight_decay

    def _update(self, key, p, g):
        st = self.state.get(key)
        if st is None or st["m"].numel() != g.numel():
            st = {"m": torch.zeros_like(p, dtype=torch.float32),
                  "v": torch.zeros_like(p, dtype=torch.float32), "t": 0}
            self.state[key] = st
        st["t"] += 1
        gf = g.float()
        st["m"].mul_(self.beta1).add_(gf, alpha=1 - self.beta1)
        st["v"].mul_(self.beta2).addcmul_(gf, gf, value=1 - self.beta2)
        mhat = st["m"] / (1 - self.beta1 ** st["t"])
        vhat = st["v"] / (1 - self.beta2 ** st["t"])
        upd = mhat / (vhat.sqrt() + self.eps) + self.weight_decay * p.float()
        p.sub_((self.lr * upd).to(p.dtype))


def _set_hyperparams(self, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float) -> None:
    self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay


def _zero_state(self) -> None:
    """Drop the moments and the step count, keep the hyper-parameters (legacy/src/momijo/learn/optim/adam.mojo:246-251)."""
    self.state.clear()
    if hasattr(self, "t"):
        self.t = 0


Adam.set_hyperparams, Adam.zero_state = _set_hyperparams, _zero_state
