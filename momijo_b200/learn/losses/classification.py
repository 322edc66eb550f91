"""List-typed classification losses (legacy/src/momijo/learn/losses/classification.mojo:120-357)."""
import math

import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def softmax_list(logits):
    return torch.softmax(_t(logits), -1).tolist()


def cross_entropy(logits, target, reduction="mean"):
    """``logits``: [N][C] (list or tensor); ``target``: class indices or one-hot rows."""
    lg = _t(logits).float() if isinstance(logits, torch.Tensor) else _t(logits)
    tg = _t(target)
    logp = torch.log_softmax(lg, -1)
    if tg.dim() == lg.dim():
        loss = -(tg.to(logp.dtype) * logp).sum(-1)
    else:
        loss = -logp.gather(-1, tg.long().unsqueeze(-1)).squeeze(-1)
    r = loss.mean() if reduction == "mean" else (loss.sum() if reduction == "sum" else loss)
    return r if isinstance(logits, torch.Tensor) else (r.tolist() if r.dim() else float(r))


def binary_cross_entropy(probs, target, eps=1e-12, reduction="mean"):
    p = _t(probs).clamp(eps, 1 - eps)
    t = _t(target).to(p.dtype)
    loss = -(t * p.log() + (1 - t) * (1 - p).log())
    r = loss.mean() if reduction == "mean" else (loss.sum() if reduction == "sum" else loss)
    return r if isinstance(probs, torch.Tensor) else (r.tolist() if r.dim() else float(r))


def hinge(scores, target, reduction="mean"):
    """target in {-1, +1}."""
    s, t = _t(scores), _t(target)
    loss = (1 - t * s).clamp_min(0)
    r = loss.mean() if reduction == "mean" else (loss.sum() if reduction == "sum" else loss)
    return r if isinstance(scores, torch.Tensor) else (r.tolist() if r.dim() else float(r))


def focal_loss(probs, target, gamma=2.0, alpha=0.25, eps=1e-12):
    p, t = _t(probs).clamp(eps, 1 - eps), _t(target)
    pt = p * t + (1 - p) * (1 - t)
    a = alpha * t + (1 - alpha) * (1 - t)
    r = (-a * (1 - pt) ** gamma * pt.log()).mean()
    return r if isinstance(probs, torch.Tensor) else float(r)


def label_smoothing_cross_entropy(logits, target, smoothing=0.1):
    lg = _t(logits)
    n = lg.shape[-1]
    logp = torch.log_softmax(lg, -1)
    tg = _t(target).long()
    nll = -logp.gather(-1, tg.unsqueeze(-1)).squeeze(-1)
    r = ((1 - smoothing) * nll + smoothing * (-logp.mean(-1))).mean()
    return r if isinstance(logits, torch.Tensor) else float(r)


def focal_loss_binary_with_logits(logits, targets, gamma=2.0, alpha=0.25):
    """Binary focal loss on logits: w * (1 - p_t)^gamma * BCE, w = alpha for targets equal to 1 and
    1 - alpha otherwise, averaged (legacy/src/momijo/learn/losses/classification.mojo:193-214, 339-345)."""
    x, y = _t(logits).double(), _t(targets).double().clamp(0, 1)
    if x.numel() == 0:
        return 0.0
    p = torch.sigmoid(x)
    pos = y == 1.0
    pt = torch.where(pos, p, 1 - p)
    w = torch.where(pos, torch.full_like(p, alpha), torch.full_like(p, 1 - alpha))
    ce = torch.nn.functional.binary_cross_entropy_with_logits(x, y, reduction="none")
    return float((w * (1 - pt) ** gamma * ce).mean())


def focal_loss_multiclass_with_logits(logits, target, gamma=2.0, alpha=0.25):
    """Multi-class focal loss on [N, C] logits; ``target`` is either N class indices or an [N, C] one-hot
    matrix (every non-zero entry contributes). One alpha for all classes, sum divided by N
    (legacy/src/momijo/learn/losses/classification.mojo:216-260, 348-363)."""
    lg = _t(logits).double()
    if lg.numel() == 0:
        return 0.0
    probs = torch.softmax(lg, -1)
    tg = _t(target)
    eps = 1e-12
    term = alpha * (1 - probs) ** gamma * (-(probs.clamp(eps, 1.0)).log())
    if tg.dim() == 1:
        picked = term.gather(-1, tg.long().unsqueeze(-1)).squeeze(-1)
        return float(picked.sum() / lg.shape[0])
    return float((term * (tg != 0)).sum() / lg.shape[0])
