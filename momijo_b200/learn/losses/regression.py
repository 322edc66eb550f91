"""Regression losses for lists and tensors (legacy/src/momijo/learn/losses/regression.mojo:122-412)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def _out(r, like):
    return r if isinstance(like, torch.Tensor) else (r.tolist() if r.dim() else float(r))


def _red(x, reduction, sample_weight=None):
    """``sample_weight`` scales each element; the weighted mean divides by the weight sum
    (legacy/src/momijo/learn/losses/regression.mojo:143-185)."""
    if sample_weight is not None:
        w = _t(sample_weight).to(x.dtype)
        x = x * w
        if reduction == "mean":
            return x.sum() / w.sum().clamp_min(1e-300)
    return x.mean() if reduction == "mean" else (x.sum() if reduction == "sum" else x)


def mse_loss(pred, target, reduction="mean", sample_weight=None):
    return _out(_red((_t(pred) - _t(target)) ** 2, reduction, sample_weight), pred)


def mae_loss(pred, target, reduction="mean", sample_weight=None):
    return _out(_red((_t(pred) - _t(target)).abs(), reduction, sample_weight), pred)


def rmse_loss(pred, target):
    return _out(((_t(pred) - _t(target)) ** 2).mean().sqrt(), pred)


def huber_loss(pred, target, delta=1.0, reduction="mean", sample_weight=None):
    d = (_t(pred) - _t(target)).abs()
    return _out(_red(torch.where(d <= delta, 0.5 * d * d, delta * (d - 0.5 * delta)), reduction, sample_weight), pred)


def smooth_l1_loss(pred, target, beta=1.0, reduction="mean"):
    d = (_t(pred) - _t(target)).abs()
    return _out(_red(torch.where(d < beta, 0.5 * d * d / beta, d - 0.5 * beta), reduction), pred)


def log_cosh_loss(pred, target, reduction="mean"):
    d = _t(pred) - _t(target)
    return _out(_red(d + torch.nn.functional.softplus(-2 * d) - 0.6931471805599453, reduction), pred)


def quantile_loss(pred, target, q=0.5, reduction="mean"):
    d = _t(target) - _t(pred)
    return _out(_red(torch.maximum(q * d, (q - 1) * d), reduction), pred)


def msle_loss(pred, target, reduction="mean"):
    return _out(_red((torch.log1p(_t(pred).clamp_min(0)) - torch.log1p(_t(target).clamp_min(0))) ** 2, reduction), pred)


def mape_loss(pred, target, eps=1e-12, reduction="mean"):
    t = _t(target)
    return _out(_red(((_t(pred) - t) / t.abs().clamp_min(eps)).abs(), reduction), pred)
