"""Distributions with ``sample / log_prob (+_tensor)``
(legacy/src/momijo/learn/prob/distributions.mojo:133-566). Sampling uses the seeded ``RNG`` of
``utils.randomness`` so results are reproducible from the seed alone."""
from __future__ import annotations

import math

import torch

from ..utils.randomness import RNG


class _Dist:
    def __init__(self, seed: int = 0):
        self.rng = RNG(seed)

    def sample_n(self, n: int):
        return [self.sample() for _ in range(n)]

    def sample_tensor(self, shape):
        n = 1
        for s in shape:
            n *= s
        return torch.tensor(self.sample_n(n), dtype=torch.float32).reshape(list(shape))

    def log_prob_tensor(self, x: torch.Tensor) -> torch.Tensor:
        return torch.tensor([self.log_prob(float(v)) for v in x.reshape(-1)], dtype=torch.float32).reshape(x.shape)

    def mean_value(self) -> float:
        """The reference's name for the mean (distributions.mojo:161, 225, 323, 428, 537)."""
        return self.mean()


class Uniform(_Dist):
    def __init__(self, low=0.0, high=1.0, seed=0):
        super().__init__(seed)
        self.low, self.high = low, high

    def sample(self):
        return self.rng.uniform(self.low, self.high)

    def log_prob(self, x):
        return -math.log(self.high - self.low) if self.low <= x <= self.high else -math.inf

    def mean(self):
        return 0.5 * (self.low + self.high)

    def variance(self):
        return (self.high - self.low) ** 2 / 12.0

    def entropy(self):
        return math.log(self.high - self.low)

    def log_prob_tensor(self, x):
        inside = (x >= self.low) & (x <= self.high)
        return torch.where(inside, torch.full_like(x, -math.log(self.high - self.low), dtype=torch.float32),
                           torch.full_like(x, -math.inf, dtype=torch.float32))


class Bernoulli(_Dist):
    def __init__(self, p=0.5, seed=0):
        super().__init__(seed)
        self.p = p

    def sample(self):
        return 1 if self.rng.bernoulli(self.p) else 0

    def log_prob(self, x):
        p = min(max(self.p, 1e-12), 1 - 1e-12)
        return math.log(p) if x >= 0.5 else math.log(1 - p)

    def mean(self):
        return self.p

    def variance(self):
        return self.p * (1 - self.p)

    def entropy(self):
        p = min(max(self.p, 1e-12), 1 - 1e-12)
        return -(p * math.log(p) + (1 - p) * math.log(1 - p))


class Binomial(_Dist):
    def __init__(self, n=1, p=0.5, seed=0):
        super().__init__(seed)
        self.n, self.p = n, p

    def sample(self):
        return sum(1 for _ in range(self.n) if self.rng.bernoulli(self.p))

    def log_prob(self, k):
        k = int(k)
        if k < 0 or k > self.n:
            return -math.inf
        p = min(max(self.p, 1e-12), 1 - 1e-12)
        return (math.lgamma(self.n + 1) - math.lgamma(k + 1) - math.lgamma(self.n - k + 1)
                + k * math.log(p) + (self.n - k) * math.log(1 - p))

    def mean(self):
        return self.n * self.p

    def variance(self):
        return self.n * self.p * (1 - self.p)


class Categorical(_Dist):
    def __init__(self, probs, seed=0):
        super().__init__(seed)
        s = float(sum(probs))
        self.probs = [p / s for p in probs]

    def sample(self):
        return self.rng.weighted_choice(self.probs)

    def log_prob(self, k):
        k = int(k)
        return math.log(max(self.probs[k], 1e-300)) if 0 <= k < len(self.probs) else -math.inf

    def entropy(self):
        return -sum(p * math.log(p) for p in self.probs if p > 0)

    # Mean and variance of a class index mean nothing: NaN, as in the reference (distributions.mojo:428-434).
    def mean(self):
        return math.nan

    def variance(self):
        return math.nan

    @staticmethod
    def from_probs_tensor(probs_t, seed=0) -> "Categorical":
        """From a 1-D tensor of weights: negatives count as 0, the rest is normalised; all-zero weights give the
        uniform distribution (distributions.mojo:445-470)."""
        ps = [max(float(v), 0.0) for v in probs_t.reshape(-1)]
        if sum(ps) <= 0.0:
            ps = [1.0] * len(ps)
        return Categorical(ps, seed)


class Normal(_Dist):
    def __init__(self, mean=0.0, std=1.0, seed=0):
        super().__init__(seed)
        self.mu, self.std = mean, std

    def sample(self):
        return self.rng.normal(self.mu, self.std)

    def log_prob(self, x):
        z = (x - self.mu) / self.std
        return -0.5 * z * z - math.log(self.std) - 0.5 * math.log(2 * math.pi)

    def log_prob_tensor(self, x):
        z = (x.float() - self.mu) / self.std
        return -0.5 * z * z - math.log(self.std) - 0.5 * math.log(2 * math.pi)

    def mean(self):
        return self.mu

    def variance(self):
        return self.std ** 2

    def entropy(self):
        return 0.5 * math.log(2 * math.pi * math.e * self.std ** 2)


def ln(x: float) -> float:
    """Natural log; -inf for non-positive input (legacy/src/momijo/learn/prob/distributions.mojo:54-65)."""
    return math.log(x) if x > 0.0 else float("-inf")


def sqrt(x: float) -> float:
    """Square root; 0.0 for non-positive input (legacy/src/momijo/learn/prob/distributions.mojo:67-75)."""
    return math.sqrt(x) if x > 0.0 else 0.0
