"""Ranking losses (legacy/src/momijo/learn/losses/ranking.mojo:97-276)."""
import torch


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.float64)


def _out(r, like):
    return r if isinstance(like, torch.Tensor) else float(r)


def margin_ranking_loss(x1, x2, y, margin=0.0):
    return _out((-_t(y) * (_t(x1) - _t(x2)) + margin).clamp_min(0).mean(), x1)


def pairwise_hinge_loss(pos, neg, margin=1.0):
    return _out((margin - _t(pos) + _t(neg)).clamp_min(0).mean(), pos)


def pairwise_logistic_loss(pos, neg):
    return _out(torch.nn.functional.softplus(-(_t(pos) - _t(neg))).mean(), pos)


def triplet_margin_loss(anchor, positive, negative, margin=1.0):
    a, p, n = _t(anchor), _t(positive), _t(negative)
    dp, dn = (a - p).pow(2).sum(-1).sqrt(), (a - n).pow(2).sum(-1).sqrt()
    return _out((dp - dn + margin).clamp_min(0).mean(), anchor)


def contrastive_loss(x1, x2, y, margin=1.0):
    d = (_t(x1) - _t(x2)).pow(2).sum(-1).sqrt()
    yy = _t(y)
    return _out((yy * d ** 2 + (1 - yy) * (margin - d).clamp_min(0) ** 2).mean() * 0.5, x1)


def listnet_loss(scores, relevance):
    p_true = torch.softmax(_t(relevance), -1)
    return _out(-(p_true * torch.log_softmax(_t(scores), -1)).sum(-1).mean(), scores)


def _reduce_list(v, reduction):
    if v.numel() == 0:
        return v.new_zeros(())
    if reduction == "sum":
        return v.sum()
    if reduction == "none":
        return v
    return v.mean()


def _sign_labels(labels):
    """{0, 1} -> {-1, +1}; anything positive counts as +1 (legacy/src/momijo/learn/losses/ranking.mojo:41-49)."""
    y = _t(labels)
    return torch.where(y > 0, torch.ones_like(y, dtype=torch.float64), -torch.ones_like(y, dtype=torch.float64))


def hinge_loss(scores, labels, margin=1.0, reduction="mean"):
    """max(0, margin - y * s) with labels mapped to +-1 (legacy/src/momijo/learn/losses/ranking.mojo:97-115)."""
    s = _t(scores)
    y = _sign_labels(labels).to(s.dtype)
    return _out(_reduce_list((margin - y * s).clamp_min(0), reduction), scores)


def triplet_loss(anchors, positives, negatives, margin=1.0, reduction="mean"):
    """max(0, ||a-p|| - ||a-n|| + margin) per row of [N, D] embeddings
    (legacy/src/momijo/learn/losses/ranking.mojo:124-152)."""
    a, p, n = _t(anchors), _t(positives), _t(negatives)
    d_ap, d_an = (a - p).pow(2).sum(-1).sqrt(), (a - n).pow(2).sum(-1).sqrt()
    return _out(_reduce_list((d_ap - d_an + margin).clamp_min(0), reduction), anchors)


def triplet_loss_from_dist(ap_dists, an_dists, margin=1.0, reduction="mean"):
    """Same from precomputed distances (legacy/src/momijo/learn/losses/ranking.mojo:160-182)."""
    return _out(_reduce_list((_t(ap_dists) - _t(an_dists) + margin).clamp_min(0), reduction), ap_dists)
