"""General metrics (legacy/src/momijo/learn/metrics/metrics.mojo:49-107)."""
import math

import torch

from .classification import precision_recall_f1  # noqa: F401


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def accuracy_approx(pred, target, tol: float = 0.5) -> float:
    """Fraction of predictions within ``tol`` of the target."""
    return float(((_t(pred) - _t(target)).abs() < tol).float().mean())


def iou(pred_mask, target_mask, eps=1e-12) -> float:
    p, t = _t(pred_mask) > 0, _t(target_mask) > 0
    return float((p & t).sum()) / (float((p | t).sum()) + eps)


def psnr(a, b, max_val=1.0, eps=0.0) -> float:
    """``eps`` is added to the mean squared error like the reference's 1e-12 (metrics.mojo:96-103); with the default 0
    identical images give ``inf``."""
    mse = float(((_t(a).double() - _t(b).double()) ** 2).mean()) + eps
    return float("inf") if mse == 0 else 10.0 * math.log10(max_val * max_val / mse)


def ssim(a, b, k1=0.01, k2=0.03, win=11, max_val=1.0) -> float:
    """Global (single-window) structural similarity; ``win`` is accepted for the reference's signature
    (metrics.mojo:107-125) and unused, as there."""
    if k1 >= 1.0 and k2 == 0.03:                 # ssim(a, b, max_val) of earlier callers
        max_val, k1 = k1, 0.01
    x, y = _t(a).double(), _t(b).double()
    c1, c2 = (k1 * max_val) ** 2, (k2 * max_val) ** 2
    mx, my = x.mean(), y.mean()
    vx, vy = x.var(unbiased=False), y.var(unbiased=False)
    cov = ((x - mx) * (y - my)).mean()
    return float((2 * mx * my + c1) * (2 * cov + c2) / ((mx * mx + my * my + c1) * (vx + vy + c2)))
