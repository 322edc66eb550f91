"""KL divergences (legacy/src/momijo/learn/prob/kl_losses.mojo:138-405)."""
import math

import torch


def kl_normal_normal(mu_p, std_p, mu_q, std_q):
    """KL(N(mu_p, std_p) || N(mu_q, std_q)); scalars or tensors."""
    if isinstance(mu_p, torch.Tensor):
        return torch.log(std_q / std_p) + (std_p ** 2 + (mu_p - mu_q) ** 2) / (2 * std_q ** 2) - 0.5
    return math.log(std_q / std_p) + (std_p ** 2 + (mu_p - mu_q) ** 2) / (2 * std_q ** 2) - 0.5


def kl_normal_standard(mu, logvar):
    """KL(N(mu, exp(logvar)) || N(0, 1)) summed over the last dim (VAE term)."""
    return -0.5 * (1 + logvar - mu ** 2 - logvar.exp()).sum(-1)


def kl_bernoulli_bernoulli(p, q, eps=1e-12):
    if isinstance(p, torch.Tensor):
        p, q = p.clamp(eps, 1 - eps), q.clamp(eps, 1 - eps)
        return p * (p / q).log() + (1 - p) * ((1 - p) / (1 - q)).log()
    p, q = min(max(p, eps), 1 - eps), min(max(q, eps), 1 - eps)
    return p * math.log(p / q) + (1 - p) * math.log((1 - p) / (1 - q))


def kl_categorical_categorical(p, q, eps=1e-12):
    pt = p if isinstance(p, torch.Tensor) else torch.tensor(p, dtype=torch.float64)
    qt = q if isinstance(q, torch.Tensor) else torch.tensor(q, dtype=torch.float64)
    r = (pt * ((pt.clamp_min(eps)) / qt.clamp_min(eps)).log()).sum(-1)
    return r if isinstance(p, torch.Tensor) else float(r)


def kl_uniform_uniform(a1, b1, a2, b2):
    if a2 <= a1 and b1 <= b2:
        return math.log((b2 - a2) / (b1 - a1))
    return math.inf


def kl_div_loss(log_q, p, reduction="batchmean"):
    """sum p * (log p - log_q)."""
    x = torch.where(p > 0, p * (p.clamp_min(1e-38).log() - log_q), torch.zeros_like(p))
    if reduction == "batchmean":
        return x.sum() / p.shape[0]
    return x.sum() if reduction == "sum" else (x.mean() if reduction == "mean" else x)


def js_divergence(p, q, eps=1e-12):
    m = 0.5 * (p + q)
    return 0.5 * kl_categorical_categorical(p, m, eps) + 0.5 * kl_categorical_categorical(q, m, eps)
