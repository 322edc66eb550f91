"""Classification metrics (legacy/src/momijo/learn/metrics/classification.mojo:64-192)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x)


def accuracy(pred, target, axis: int = -1) -> float:
    """``pred`` may be class indices or scores with the classes along ``axis``."""
    p, t = _t(pred), _t(target)
    if p.dim() == t.dim() + 1:
        p = p.argmax(axis)
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


def argmax_index(xs) -> int:
    """Index of the first maximum of a list (legacy/src/momijo/learn/metrics/classification.mojo:38-48)."""
    best_idx, best_val = 0, -1.7976931348623157e308
    for i, v in enumerate(xs):
        if v > best_val:
            best_idx, best_val = i, v
    return best_idx


def confusion_matrix_from_labels(y_pred, y_true, n_classes: int):
    """Rows = true class, columns = predicted class; labels outside [0, n_classes) are skipped
    (legacy/src/momijo/learn/metrics/classification.mojo:64-84). Returns nested lists."""
    cm = [[0] * n_classes for _ in range(n_classes)]
    for p, t in zip(list(y_pred), list(y_true)):
        p, t = int(p), int(t)
        if 0 <= t < n_classes and 0 <= p < n_classes:
            cm[t][p] += 1
    return cm


def f1_score_binary(y_pred, y_true, threshold: float = 0.5) -> float:
    """F1 of thresholded scores against {0, 1} labels; 0.0 on empty or mismatched inputs
    (legacy/src/momijo/learn/metrics/classification.mojo:121-145)."""
    y_pred, y_true = list(y_pred), list(y_true)
    if len(y_true) == 0 or len(y_true) != len(y_pred):
        return 0.0
    tp = fp = fn = 0
    for s, yt in zip(y_pred, y_true):
        yhat = 1 if float(s) >= threshold else 0
        yt = int(yt)
        if yhat == 1 and yt == 1:
            tp += 1
        elif yhat == 1 and yt == 0:
            fp += 1
        elif yhat == 0 and yt == 1:
            fn += 1
    prec = tp / (tp + fp) if tp + fp else 0.0
    rec = tp / (tp + fn) if tp + fn else 0.0
    return 2 * prec * rec / (prec + rec) if prec + rec else 0.0
