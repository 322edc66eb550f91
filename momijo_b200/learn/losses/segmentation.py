"""Segmentation losses (legacy/src/momijo/learn/losses/segmentation.mojo:61-305)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def _out(r, like):
    return r if isinstance(like, torch.Tensor) else float(r)


def dice_loss(probs, target, eps=1e-6):
    p, t = _t(probs), _t(target)
    return _out(1 - (2 * (p * t).sum() + eps) / (p.sum() + t.sum() + eps), probs)


def iou_loss(probs, target, eps=1e-6):
    p, t = _t(probs), _t(target)
    inter = (p * t).sum()
    return _out(1 - (inter + eps) / (p.sum() + t.sum() - inter + eps), probs)


jaccard_loss = iou_loss


def tversky_loss(probs, target, alpha=0.5, beta=0.5, eps=1e-6):
    p, t = _t(probs), _t(target)
    tp, fp, fn = (p * t).sum(), (p * (1 - t)).sum(), ((1 - p) * t).sum()
    return _out(1 - (tp + eps) / (tp + alpha * fp + beta * fn + eps), probs)


def focal_tversky_loss(probs, target, alpha=0.5, beta=0.5, gamma=0.75, eps=1e-6):
    tv = _t(tversky_loss(_t(probs), _t(target), alpha, beta, eps))
    return _out(tv ** gamma, probs)


def bce_dice_loss(probs, target, eps=1e-12):
    p, t = _t(probs).clamp(eps, 1 - eps), _t(target)
    bce = -(t * p.log() + (1 - t) * (1 - p).log()).mean()
    return _out(bce + _t(dice_loss(p, t)), probs)


def dice_loss_mc_vec(preds_per_class, targets_per_class, eps=1e-6):
    """Per-class binary Dice losses (legacy/src/momijo/learn/losses/segmentation.mojo:112-121, 223-232)."""
    assert len(preds_per_class) == len(targets_per_class)
    return [float(dice_loss(_t(p).clamp(0, 1), _t(t).clamp(0, 1), eps))
            for p, t in zip(preds_per_class, targets_per_class)]


def iou_loss_mc_vec(preds_per_class, targets_per_class, eps=1e-6):
    assert len(preds_per_class) == len(targets_per_class)
    return [float(iou_loss(_t(p).clamp(0, 1), _t(t).clamp(0, 1), eps))
            for p, t in zip(preds_per_class, targets_per_class)]


def _mc_reduce(vec, reduction):
    if not vec:
        return 0.0
    return float(sum(vec)) if reduction == "sum" else float(sum(vec) / len(vec))   # "none" also averages


def dice_loss_mc(preds_per_class, targets_per_class, eps=1e-6, reduction="mean"):
    """Mean (or sum) of the per-class Dice losses; ``reduction="none"`` averages too, as in the reference
    (legacy/src/momijo/learn/losses/segmentation.mojo:134-144)."""
    return _mc_reduce(dice_loss_mc_vec(preds_per_class, targets_per_class, eps), reduction)


def iou_loss_mc(preds_per_class, targets_per_class, eps=1e-6, reduction="mean"):
    return _mc_reduce(iou_loss_mc_vec(preds_per_class, targets_per_class, eps), reduction)
