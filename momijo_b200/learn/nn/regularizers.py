"""L1 / L2 / elastic-net penalties for lists and tensors
(legacy/src/momijo/learn/nn/regularizers.mojo:68-247)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def l1_penalty(w, lam=1.0):
    r = lam * _t(w).abs().sum()
    return r if isinstance(w, torch.Tensor) else float(r)


def l2_penalty(w, lam=1.0):
    r = 0.5 * lam * (_t(w) ** 2).sum()
    return r if isinstance(w, torch.Tensor) else float(r)


def elastic_net_penalty(w, l1=1.0, l2=1.0):
    return l1_penalty(w, l1) + l2_penalty(w, l2)


def l1_grad(w, lam=1.0):
    r = lam * torch.sign(_t(w))
    return r if isinstance(w, torch.Tensor) else r.tolist()


def l2_grad(w, lam=1.0):
    r = lam * _t(w)
    return r if isinstance(w, torch.Tensor) else r.tolist()


def elastic_net_grad(w, l1=1.0, l2=1.0):
    r = l1 * torch.sign(_t(w)) + l2 * _t(w)
    return r if isinstance(w, torch.Tensor) else r.tolist()


def apply_weight_decay_(w, lr, lam):
    """Decoupled decay: w <- w * (1 - lr * lam)."""
    with torch.no_grad():
        return w.mul_(1.0 - lr * lam)
