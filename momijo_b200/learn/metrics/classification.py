"""Classification metrics (legacy/src/momijo/learn/metrics/classification.mojo:64-192)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x)


def accuracy(pred, target) -> float:
    """``pred`` may be class indices or [N, C] scores."""
    p, t = _t(pred), _t(target)
    if p.dim() == t.dim() + 1:
        p = p.argmax(-1)
    return float((p == t).float().mean()) if p.numel() else 0.0


def confusion_matrix(pred, target, num_classes: int):
    p, t = _t(pred).long().reshape(-1), _t(target).long().reshape(-1)
    cm = torch.zeros(num_classes, num_classes, dtype=torch.int64)
    cm.index_put_((t, p), torch.ones_like(t), accumulate=True)
    return cm


def precision_recall_f1(pred, target, positive=1, eps=1e-12):
    p, t = _t(pred), _t(target)
    tp = float(((p == positive) & (t == positive)).sum())
    fp = float(((p == positive) & (t != positive)).sum())
    fn = float(((p != positive) & (t == positive)).sum())
    pr, rc = tp / (tp + fp + eps), tp / (tp + fn + eps)
    return pr, rc, 2 * pr * rc / (pr + rc + eps)


def f1_score(pred, target, average="binary", num_classes=None, positive=1) -> float:
    if average == "binary":
        return precision_recall_f1(pred, target, positive)[2]
    p, t = _t(pred), _t(target)
    k = num_classes or int(max(p.max(), t.max())) + 1
    f1s, sup = [], []
    for c in range(k):
        f1s.append(precision_recall_f1(p, t, c)[2])
        sup.append(float((t == c).sum()))
    if average == "macro":
        return sum(f1s) / k
    if average == "weighted":
        return sum(f * s for f, s in zip(f1s, sup)) / max(sum(sup), 1.0)
    cm = confusion_matrix(p, t, k)  # micro
    return float(cm.diag().sum()) / max(float(cm.sum()), 1.0)
