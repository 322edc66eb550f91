"""Flat-buffer optimizer kernels: fused AdamW / SGD over fp32 master shards and the squared
gradient norm with non-finite detection (feeds GradScaler and clipping)."""
from __future__ import annotations

import torch

from .. import _C


def adamw_flat(grad, master, m, v, param_out, *, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale=1.0, grad_scale_dev=None, found_inf=None):
    """One AdamW step on flat tensors. ``grad`` bf16 or fp32; ``master/m/v`` fp32;
    ``param_out`` (bf16, optional) receives the rounded parameters."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    n = master.numel()
    if not master.is_cuda:
        g = grad.float() * grad_scale
        if grad_scale_dev is not None:
            g = g * grad_scale_dev.float()
        if found_inf is not None and int(found_inf) != 0:
            return
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        upd = (m / bc1) / ((v / bc2).sqrt() + eps)
        master.sub_(lr * (upd + weight_decay * master))
        if param_out is not None:
            param_out.copy_(master.to(param_out.dtype))
        return
    _C.call("mmj_adamw", _C.ptr(grad), 0 if grad.dtype == torch.bfloat16 else 1, _C.ptr(master),
            _C.ptr(m), _C.ptr(v), _C.ptr(param_out), n, lr, beta1, beta2, eps, weight_decay, bc1,
            bc2, grad_scale, _C.ptr(grad_scale_dev), _C.ptr(found_inf), _C.current_stream())


def sgd_flat(grad, master, momentum_buf, param_out, *, lr, momentum=0.0, weight_decay=0.0,
             grad_scale=1.0):
    n = master.numel()
    if not master.is_cuda:
        g = grad.float() * grad_scale + weight_decay * master
        if momentum_buf is not None:
            momentum_buf.mul_(momentum).add_(g)
            g = momentum_buf
        master.sub_(lr * g)
        if param_out is not None:
            param_out.copy_(master.to(param_out.dtype))
        return
    _C.call("mmj_sgd", _C.ptr(grad), 0 if grad.dtype == torch.bfloat16 else 1, _C.ptr(master),
            _C.ptr(momentum_buf), _C.ptr(param_out), n, lr, momentum, weight_decay, grad_scale,
            _C.current_stream())


def sq_norm(x, out=None, found_inf=None, accumulate=False):
    """Sum of squares of ``x`` into ``out[0]`` (fp32); sets ``found_inf[0]`` on inf/nan."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        s = x.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s
        if found_inf is not None and not torch.isfinite(x.float()).all():
            found_inf[0] = 1
        return out
    parts = _C.lib().mmj_sqnorm_parts()
    scratch = torch.empty(parts, dtype=torch.float32, device=x.device)
    _C.call("mmj_sqnorm", _C.ptr(x), 0 if x.dtype == torch.bfloat16 else 1, x.numel(),
            _C.ptr(scratch), _C.ptr(out), _C.ptr(found_inf), int(accumulate), _C.current_stream())
    return out
