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


def psnr(a, b, max_val=1.0) -> float:
    mse = float(((_t(a).double() - _t(b).double()) ** 2).mean())
    return float("inf") if mse == 0 else 10.0 * math.log10(max_val * max_val / mse)


def ssim(a, b, max_val=1.0) -> float:
    """Global (single-window) structural similarity."""
    x, y = _t(a).double(), _t(b).double()
    c1, c2 = (0.01 * max_val) ** 2, (0.03 * max_val) ** 2
    mx, my = x.mean(), y.mean()
    vx, vy = x.var(unbiased=False), y.var(unbiased=False)
    cov = ((x - mx) * (y - my)).mean()
    return float((2 * mx * my + c1) * (2 * cov + c2) / ((mx * mx + my * my + c1) * (vx + vy + c2)))
