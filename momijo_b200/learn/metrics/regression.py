"""Regression metrics (legacy/src/momijo/learn/metrics/regression.mojo:88-189)."""
import torch


def _t(x):
    return (x if isinstance(x, torch.Tensor) else torch.tensor(x)).double()


def mse(pred, target):
    return float(((_t(pred) - _t(target)) ** 2).mean())


def rmse(pred, target):
    return mse(pred, target) ** 0.5


def mae(pred, target):
    return float((_t(pred) - _t(target)).abs().mean())


def mape(pred, target, scale=1.0, eps=1e-12):
    """Mean absolute relative error times ``scale`` (the reference's default scale is 100, a percentage; this
    package's default stays a fraction). A small second positional value is read as ``eps`` for earlier callers."""
    if scale < 1e-3:
        scale, eps = 1.0, scale
    t = _t(target)
    return float(((_t(pred) - t).abs() / t.abs().clamp_min(eps)).mean()) * scale


def r2_score(pred, target):
    p, t = _t(pred), _t(target)
    ss_res = ((t - p) ** 2).sum()
    ss_tot = ((t - t.mean()) ** 2).sum()
    return float(1 - ss_res / ss_tot) if float(ss_tot) > 0 else 0.0


def explained_variance(pred, target):
    p, t = _t(pred), _t(target)
    vt = t.var(unbiased=False)
    return float(1 - (t - p).var(unbiased=False) / vt) if float(vt) > 0 else 0.0
