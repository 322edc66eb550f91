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


# ---- list / tensor-list drivers of the reference (adagrad.mojo:135-320) -----------------------------------------
def _ada_step_on_lists(self, params, grads):
    """Scalar lists: updates ``params`` in place and returns it; accumulators persist across calls."""
    if len(params) != len(grads):
        raise ValueError("Adagrad.step_on_lists: length mismatch")
    acc = self.state.setdefault("scalars", [])
    acc.extend([0.0] * (len(params) - len(acc)))
    for i in range(len(params)):
        params[i], acc[i] = adagrad_update_scalar(params[i], grads[i], acc[i], self.lr, self.eps, self.weight_decay)
    return params


def _ada_update_tensor(self, param, grad, acc):
    """Pure form: returns ``(new parameter, new accumulator)`` and leaves its inputs alone."""
    g = grad + self.weight_decay * param if self.weight_decay else grad
    acc_new = acc + g * g
    return param - self.lr * g / (acc_new.sqrt() + self.eps), acc_new


def _ada_step_on_tensor_list(self, params, grads, _slot="tensors"):
    if len(params) != len(grads):
        raise ValueError("Adagrad.step_on_tensor_list: length mismatch")
    accs = self.state.setdefault(_slot, [])
    for i in range(len(accs), len(params)):
        accs.append(torch.zeros_like(params[i]))
    with torch.no_grad():
        for i in range(len(params)):
            new_p, accs[i] = _ada_update_tensor(self, params[i], grads[i], accs[i])
            params[i] = new_p
    return params


Adagrad.step_on_lists = _ada_step_on_lists
Adagrad.adagrad_update_tensor_f32 = Adagrad.adagrad_update_tensor_f64 = _ada_update_tensor
Adagrad.step_on_tensor_list = _ada_step_on_tensor_list
Adagrad.step_on_tensor_list_f32 = lambda self, params, grads: _ada_step_on_tensor_list(self, params, grads, "tensors_f32")
Adagrad.reset_state = lambda self: self.state.clear()
