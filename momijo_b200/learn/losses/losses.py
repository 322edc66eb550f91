"""Tensor losses (legacy/src/momijo/learn/losses/losses.mojo:46-273).

``softmax_cross_entropy`` returns ``(loss, dlogits)`` in one call like the reference; on CUDA bf16
logits it is the fused kernel of ``momijo_b200.ops``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as tF

from ... import ops


def _reduce(x, reduction):
    if reduction == "mean":
        return x.mean()
    if reduction == "sum":
        return x.sum()
    return x


def cross_entropy_from_probs(probs, y_onehot, eps: float = 1e-7):
    """-sum(y * log(clip(p))) / N  (losses.mojo:46)."""
    p = probs.clamp(eps, 1.0 - eps)
    return -(y_onehot * p.log()).sum() / probs.shape[0]


def cross_entropy_from_logits(logits, y_onehot):
    return -(y_onehot * torch.log_softmax(logits.float(), -1)).sum() / logits.shape[0]


def softmax(x, axis: int = -1):
    """Row softmax (legacy/src/momijo/learn/losses/losses.mojo re-exports the tensor softmax)."""
    return torch.softmax(x.float(), axis).to(x.dtype) if x.is_floating_point() else torch.softmax(x.float(), axis)


def softmax_cross_entropy(logits, y):
    """``y`` is either one-hot ``[N, C]`` or class indices ``[N]``. Returns (loss, dlogits) with
    ``dlogits = (softmax - onehot) / N`` (losses.mojo:72-85)."""
    if y.dtype in (torch.int64, torch.int32) and y.dim() == logits.dim() - 1:
        return ops.softmax_cross_entropy(logits, y.long())
    probs = torch.softmax(logits.float(), -1)
    loss = cross_entropy_from_probs(probs, y.float())
    return loss, ((probs - y.float()) / logits.shape[0]).to(logits.dtype)


def mse(pred, target, reduction="mean"):
    return _reduce((pred - target) ** 2, reduction)


def mae(pred, target, reduction="mean"):
    return _reduce((pred - target).abs(), reduction)


def huber(pred, target, delta=1.0, reduction="mean"):
    d = (pred - target).abs()
    return _reduce(torch.where(d <= delta, 0.5 * d * d, delta * (d - 0.5 * delta)), reduction)


def smooth_l1(pred, target, beta=1.0, reduction="mean"):
    d = (pred - target).abs()
    return _reduce(torch.where(d < beta, 0.5 * d * d / beta, d - 0.5 * beta), reduction)


def bce(probs, target, eps=1e-12, reduction="mean"):
    p = probs.clamp(eps, 1 - eps)
    return _reduce(-(target * p.log() + (1 - target) * (1 - p).log()), reduction)


def bce_with_logits(logits, target, pos_weight=None, reduction="mean"):
    """Stable form max(x,0) - x*t + log1p(exp(-|x|))."""
    x = logits
    loss = x.clamp_min(0) - x * target + torch.log1p(torch.exp(-x.abs()))
    if pos_weight is not None:
        loss = loss * (1 + (pos_weight - 1) * target)
    return _reduce(loss, reduction)


def kl_div(p, q, eps: float = 1e-12, reduction: str = "sum", log_input: bool = False):
    """KL(p || q) = sum p * log(p / q) over all elements, both arguments probabilities clipped to ``[eps, 1]``
    (legacy/src/momijo/learn/losses/losses.mojo:172-177: full sum, no mean).

    ``log_input=True`` gives the other common convention instead: the first argument holds
    log-probabilities of the model and the second the target probabilities, and the result is
    ``q * (log q - log_p)`` reduced by ``reduction`` ("sum", "mean" over elements, "batchmean", "none")."""
    if log_input:
        v = torch.where(q > 0, q * (q.clamp_min(1e-38).log() - p), torch.zeros_like(q))
        if reduction == "batchmean":
            return v.sum() / v.shape[0]
        return _reduce(v, reduction)
    pp, qq = p.clamp(eps, 1.0), q.clamp(eps, 1.0)
    v = pp * (pp / qq).clamp_min(eps).log()
    if reduction == "batchmean":
        return v.sum() / v.shape[0]
    return _reduce(v, reduction)


def nll_loss(log_probs, target, class_weight=None, reduction="mean"):
    return tF.nll_loss(log_probs, target, weight=class_weight, reduction=reduction)


def cross_entropy(logits, target, class_weight=None, reduction="mean"):
    return tF.cross_entropy(logits.float(), target, weight=class_weight, reduction=reduction)


def focal(logits, target, gamma=2.0, alpha=0.25, reduction="mean"):
    p = torch.sigmoid(logits)
    ce = bce_with_logits(logits, target, reduction="none")
    pt = p * target + (1 - p) * (1 - target)
    a = alpha * target + (1 - alpha) * (1 - target)
    return _reduce(a * (1 - pt) ** gamma * ce, reduction)


def dice(probs, target, eps=1e-6):
    inter = (probs * target).sum()
    return 1.0 - (2 * inter + eps) / (probs.sum() + target.sum() + eps)


def triplet(anchor, positive, negative, margin=1.0, reduction="mean"):
    dp = (anchor - positive).pow(2).sum(-1).sqrt()
    dn = (anchor - negative).pow(2).sum(-1).sqrt()
    return _reduce((dp - dn + margin).clamp_min(0), reduction)


def cosine_embedding(a, b, y, margin=0.0, reduction="mean"):
    cos = tF.cosine_similarity(a, b, dim=-1)
    return _reduce(torch.where(y > 0, 1 - cos, (cos - margin).clamp_min(0)), reduction)


def triplet_loss(anchor, positive, negative, margin: float = 1.0):
    """max(0, sum((a-p)^2) - sum((a-n)^2) + margin) with both sums taken over every element, as the
    reference's tensor overload does (legacy/src/momijo/learn/losses/losses.mojo:257-270). The per-row
    L2 form is ``losses.ranking.triplet_loss``."""
    dap = (anchor - positive).pow(2).sum()
    dan = (anchor - negative).pow(2).sum()
    return (dap - dan + margin).clamp_min(0)


def cosine_embedding_loss(x1, x2, target, margin: float = 0.0, eps: float = 1e-12):
    """Whole-tensor cosine between x1 and x2; 1 - cos where target > 0, max(0, cos - margin) elsewhere,
    averaged over target (legacy/src/momijo/learn/losses/losses.mojo:273-290)."""
    dot = (x1 * x2).sum()
    n1 = ((x1 * x1).sum() + eps).sqrt()
    n2 = ((x2 * x2).sum() + eps).sqrt()
    cos = dot / (n1 * n2)
    return torch.where(target > 0, 1.0 - cos, (cos - margin).clamp_min(0)).mean()


# ---- the reference's tensor forms under their own names (legacy/src/momijo/learn/losses/losses.mojo:127-246) -----------
def mse_loss(pred, target, reduction="mean"):
    return mse(pred, target, reduction)


def focal_loss(logits, target_index, gamma: float = 2.0, alpha=None, axis: int = -1, eps: float = 1e-12):
    """Mean cross-entropy scaled by the batch mean of ``(1 - p_t)^gamma`` (and by ``alpha`` when given), ``p_t`` the
    softmax probability of the true class clipped to ``[eps, 1]`` (losses.mojo:206-238). ``target_index`` holds class
    indices."""
    lg = logits if isinstance(logits, torch.Tensor) else torch.tensor(logits, dtype=torch.float32)
    tg = (target_index if isinstance(target_index, torch.Tensor) else torch.tensor(target_index)).long()
    if axis not in (-1, lg.dim() - 1):
        lg = lg.movedim(axis, -1)
    sm = torch.softmax(lg.float(), -1).clamp(eps, 1.0)
    pt = sm.gather(-1, tg.unsqueeze(-1)).squeeze(-1)
    ce = -(pt.log()).mean()
    return ce * (1.0 if alpha is None else float(alpha)) * ((1.0 - pt) ** gamma).mean()


def dice_loss(pred, target, eps: float = 1e-6):
    """``1 - 2 * sum(p * t) / (sum(p) + sum(t) + eps)`` over all elements (losses.mojo:240-248)."""
    p = pred if isinstance(pred, torch.Tensor) else torch.tensor(pred, dtype=torch.float32)
    t = target if isinstance(target, torch.Tensor) else torch.tensor(target, dtype=torch.float32)
    return 1.0 - 2.0 * (p * t).sum() / (p.sum() + t.sum() + eps)
