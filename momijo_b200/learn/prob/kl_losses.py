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


# ---- the reference's explicit forms (legacy/src/momijo/learn/prob/kl_losses.mojo:138-440) ----------------
# Normals are parameterised by mean and log-variance, variances and probabilities are clamped to 1e-12
# (probabilities also to 1 - 1e-12), and negative terms (rounding) are dropped: scalar and list forms clamp
# the result at zero, tensor forms add only the positive element terms.
_EPS = 1e-12


def _clamp_prob(x):
    return min(max(float(x), _EPS), 1.0 - _EPS)


def kl_normal_normal_scalar(mu_p, logvar_p, mu_q, logvar_q) -> float:
    var_p, var_q = max(math.exp(logvar_p), _EPS), max(math.exp(logvar_q), _EPS)
    kl = 0.5 * ((logvar_q - logvar_p) + (var_p + (mu_p - mu_q) ** 2) / var_q - 1.0)
    return max(kl, 0.0)


def kl_normal_normal_diag(mu_p, logvar_p, mu_q, logvar_q) -> float:
    assert len(mu_p) == len(mu_q) == len(logvar_p) == len(logvar_q)
    return max(sum(kl_normal_normal_scalar(a, b, c, d) for a, b, c, d in zip(mu_p, logvar_p, mu_q, logvar_q)), 0.0)


def kl_bernoulli_scalar(p, q) -> float:
    pc, qc = _clamp_prob(p), _clamp_prob(q)
    kl = pc * (math.log(pc) - math.log(qc)) + (1 - pc) * (math.log(1 - pc) - math.log(1 - qc))
    return max(kl, 0.0)


def kl_bernoulli_vector(p, q) -> float:
    assert len(p) == len(q)
    return max(sum(kl_bernoulli_scalar(a, b) for a, b in zip(p, q)), 0.0)


def kl_categorical(p, q) -> float:
    assert len(p) == len(q)
    acc = 0.0
    for a, b in zip(p, q):
        pi, qi = _clamp_prob(a), _clamp_prob(b)
        acc += pi * (math.log(pi) - math.log(qi))
    return max(acc, 0.0)


def kl_divergence(p, q) -> float:
    """KL between two ``Normal`` or two ``Bernoulli`` distribution objects."""
    from .distributions import Bernoulli, Normal
    if isinstance(p, Normal) and isinstance(q, Normal):
        sp, sq = max(float(p.std), _EPS), max(float(q.std), _EPS)
        mp = p.mu if hasattr(p, "mu") else p.mean
        mq = q.mu if hasattr(q, "mu") else q.mean
        return kl_normal_normal_scalar(float(mp), 2.0 * math.log(sp), float(mq), 2.0 * math.log(sq))
    if isinstance(p, Bernoulli) and isinstance(q, Bernoulli):
        return kl_bernoulli_scalar(p.p, q.p)
    raise TypeError("kl_divergence takes two Normal or two Bernoulli distributions")


def kl_divergence_any(p, q) -> float:
    """Compatibility shim of the reference: always 0.0 (use the typed functions)."""
    return 0.0


def _raw(t):
    if isinstance(t, torch.Tensor):
        return t
    from ...tensor.tensor import _raw as unwrap
    return unwrap(t)


def _normal_terms(mu_p, logvar_p, mu_q, logvar_q):
    mu_p, logvar_p, mu_q, logvar_q = (_raw(x).double() for x in (mu_p, logvar_p, mu_q, logvar_q))
    assert mu_p.shape == mu_q.shape == logvar_p.shape == logvar_q.shape
    var_p, var_q = logvar_p.exp().clamp_min(_EPS), logvar_q.exp().clamp_min(_EPS)
    return (0.5 * ((logvar_q - logvar_p) + (var_p + (mu_p - mu_q) ** 2) / var_q - 1.0)).clamp_min(0)


def _bernoulli_terms(p, q):
    p, q = _raw(p).double().clamp(_EPS, 1 - _EPS), _raw(q).double().clamp(_EPS, 1 - _EPS)
    assert p.shape == q.shape
    return (p * (p.log() - q.log()) + (1 - p) * ((1 - p).log() - (1 - q).log())).clamp_min(0)


def _categorical_terms(p, q):
    p, q = _raw(p).double().clamp(_EPS, 1 - _EPS), _raw(q).double().clamp(_EPS, 1 - _EPS)
    assert p.shape == q.shape
    return (p * (p.log() - q.log())).clamp_min(0)


def _batched(terms, like):
    assert terms.dim() == 2, "batched forms take [N, D] inputs"
    out = terms.sum(-1).to(_raw(like).dtype)
    if isinstance(like, torch.Tensor):
        return out
    from ...tensor.tensor import _wrap
    return _wrap(out)


def kl_normal_normal_diag_sum(mu_p, logvar_p, mu_q, logvar_q) -> float:
    return float(_normal_terms(mu_p, logvar_p, mu_q, logvar_q).sum())


def kl_normal_normal_diag_batched(mu_p, logvar_p, mu_q, logvar_q):
    return _batched(_normal_terms(mu_p, logvar_p, mu_q, logvar_q), mu_p)


def kl_bernoulli_sum(p, q) -> float:
    return float(_bernoulli_terms(p, q).sum())


def kl_bernoulli_batched(p, q):
    return _batched(_bernoulli_terms(p, q), p)


def kl_categorical_sum(p, q) -> float:
    return float(_categorical_terms(p, q).sum())


def kl_categorical_batched(p, q):
    return _batched(_categorical_terms(p, q), p)
