"""L1 / L2 / elastic-net penalties for lists and tensors
(legacy/src/momijo/learn/nn/regularizers.mojo:68-247)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def l1_penalty(w, lam=1.0):
    r = lam * _t(w).abs().sum()
    return r if isinstance(w, torch.Tensor) else float(r)


def l2_penalty(w, lam=1.0, use_half_factor=True):
    """0.5 * lam * sum(w^2); ``use_half_factor=False`` drops the 0.5."""
    r = (0.5 if use_half_factor else 1.0) * lam * (_t(w) ** 2).sum()
    return r if isinstance(w, torch.Tensor) else float(r)


def elastic_net_penalty(w, l1=1.0, l2=1.0, use_half_factor=True):
    return l1_penalty(w, l1) + l2_penalty(w, l2, use_half_factor)


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


# ---- typed names of the reference (legacy/src/momijo/learn/nn/regularizers.mojo:162-253) --------------
# ``*_tensor_*`` take one tensor, ``*_tensors_*`` a list of tensors (parameter blocks); the suffix is the
# accumulation precision. All return a Python float.
def _raw(w):
    if isinstance(w, torch.Tensor):
        return w
    from ...tensor.tensor import _raw as unwrap
    return unwrap(w)


def _l1_sum(w, dt):
    return float(_raw(w).detach().to(dt).abs().sum())


def _l2_sum(w, dt):
    return float((_raw(w).detach().to(dt) ** 2).sum())


def _make(dt):
    def l1_one(w, weight):
        return 0.0 if weight == 0.0 else weight * _l1_sum(w, dt)

    def l2_one(w, weight, use_half_factor=True):
        if weight == 0.0:
            return 0.0
        return (0.5 if use_half_factor else 1.0) * weight * _l2_sum(w, dt)

    def en_one(w, l1, l2, use_half_factor=True):
        return l1_one(w, l1) + l2_one(w, l2, use_half_factor)

    def l1_many(blocks, weight):
        return 0.0 if weight == 0.0 else weight * sum(_l1_sum(b, dt) for b in blocks)

    def l2_many(blocks, weight, use_half_factor=True):
        if weight == 0.0:
            return 0.0
        return (0.5 if use_half_factor else 1.0) * weight * sum(_l2_sum(b, dt) for b in blocks)

    def en_many(blocks, l1, l2, use_half_factor=True):
        return l1_many(blocks, l1) + l2_many(blocks, l2, use_half_factor)

    return l1_one, l2_one, en_one, l1_many, l2_many, en_many


(l1_penalty_tensor_f32, l2_penalty_tensor_f32, elastic_net_penalty_tensor_f32,
 l1_penalty_tensors_f32, l2_penalty_tensors_f32, elastic_net_penalty_tensors_f32) = _make(torch.float32)
(l1_penalty_tensor_f64, l2_penalty_tensor_f64, elastic_net_penalty_tensor_f64,
 l1_penalty_tensors_f64, l2_penalty_tensors_f64, elastic_net_penalty_tensors_f64) = _make(torch.float64)
