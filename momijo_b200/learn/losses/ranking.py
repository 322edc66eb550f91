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
