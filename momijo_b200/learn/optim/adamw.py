"""``AdamW``: decoupled decay using the pre-update weight, bias decays too
(legacy/src/momijo/learn/optim/adamw.mojo:105-147). On CUDA fp32 master tensors with bf16/fp32
gradients the update is the fused kernel (``momijo_b200.ops.adamw_flat``)."""
import torch

from ... import ops
from .base import _PerLayerOptimizer


class AdamW(_PerLayerOptimizer):
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
            st = {"m": torch.zeros(p.numel(), dtype=torch.float32, device=p.device),
                  "v": torch.zeros(p.numel(), dtype=torch.float32, device=p.device), "t": 0}
            if p.dtype != torch.float32:
                st["master"] = p.detach().float().reshape(-1).clone()
            self.state[key] = st
        st["t"] += 1
        if p.is_cuda and p.is_contiguous() and g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16):
            master = st.get("master", p.data.view(-1))
            out = p.data.view(-1) if p.dtype == torch.bfloat16 else None
            ops.adamw_flat(g.reshape(-1), master, st["m"], st["v"], out, lr=self.lr, beta1=self.beta1,
                           beta2=self.beta2, eps=self.eps, weight_decay=self.weight_decay, step=st["t"])
            return
        gf = g.float().reshape(-1)
        st["m"].mul_(self.beta1).add_(gf, alpha=1 - self.beta1)
        st["v"].mul_(self.beta2).addcmul_(gf, gf, value=1 - self.beta2)
        mhat = st["m"] / (1 - self.beta1 ** st["t"])
        vhat = st["v"] / (1 - self.beta2 ** st["t"])
        w = st.get("master", p.data.view(-1).float() if p.dtype != torch.float32 else p.data.view(-1))
        w.sub_(self.lr * (mhat / (vhat.sqrt() + self.eps) + self.weight_decay * w))
        if "master" in st or p.dtype != torch.float32:
            p.data.copy_(w.view(p.shape).to(p.dtype))


def _set_hyperparams(self, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float) -> None:
    self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay


def _zero_state(self) -> None:
    """Drop the moments and the step count, keep the hyper-parameters (legacy/src/momijo/learn/optim/adamw.mojo:246-251)."""
    self.state.clear()
    if hasattr(self, "t"):
        self.t = 0


AdamW.set_hyperparams, AdamW.zero_state = _set_hyperparams, _zero_state
