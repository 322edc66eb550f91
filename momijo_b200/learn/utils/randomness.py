"""Seeded generators (legacy/src/momijo/learn/utils/randomness.mojo:36-450): ``SplitMix64``,
``Xoshiro256ss`` (+ ``jump``), ``RNG`` (uniform / normal / randint / bernoulli / shuffle /
permutation / choice_k / weighted_choice), ``SeedBundle``, ``seed_all``, ``derived_rngs``."""
from __future__ import annotations

import math
from dataclasses import dataclass

M64 = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int = 0):
        self.state = seed & M64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    next = next_u64


def _rotl(x, k):
    return ((x << k) | (x >> (64 - k))) & M64


class Xoshiro256ss:
    def __init__(self, seed: int = 0):
        sm = SplitMix64(seed)
        self.s = [sm.next_u64() for _ in range(4)]

    @staticmethod
    def from_seed(seed: int) -> "Xoshiro256ss":
        """State from four SplitMix64 draws; an all-zero state gets its last word set to 1
        (legacy/src/momijo/learn/utils/randomness.mojo:92-101)."""
        g = Xoshiro256ss(seed)
        if not any(g.s):
            g.s[3] = 1
        return g

    def next_u64(self) -> int:
        s = self.s
        result = (_rotl((s[1] * 5) & M64, 7) * 9) & M64
        t = (s[1] << 17) & M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def jump(self):
        """Advance by 2^128 steps (independent streams)."""
        J = [0x180EC6D33CFD0ABA, 0xD5A61266F0C9392C, 0xA9582618E03FC9AA, 0x39ABDC4529B1661C]
        s0 = s1 = s2 = s3 = 0
        for j in J:
            for b in range(64):
                if j & (1 << b):
                    s0 ^= self.s[0]; s1 ^= self.s[1]; s2 ^= self.s[2]; s3 ^= self.s[3]
                self.next_u64()
        self.s = [s0, s1, s2, s3]
        return self


class RNG:
    def __init__(self, seed: int = 0):
        self.gen = Xoshiro256ss(seed)
        self._spare = None

    def next_u64(self):
        return self.gen.next_u64()

    @staticmethod
    def from_int_seed(seed: int) -> "RNG":
        return RNG(int(seed) & M64)

    def next_f64_open01(self) -> float:
        """Uniform in the open interval (0, 1): the end points map to the nearest value inside."""
        y = (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)
        return 5e-324 if y <= 0.0 else (1.0 - 2.0 ** -53 if y >= 1.0 else y)

    next_f64 = next_f64_open01

    def uniform(self, lo: float = 0.0, hi: float = 1.0) -> float:
        return lo + (hi - lo) * ((self.gen.next_u64() >> 11) * (1.0 / 9007199254740992.0))

    def normal(self, mean: float = 0.0, std: float = 1.0) -> float:
        if self._spare is not None:
            z, self._spare = self._spare, None
            return mean + std * z
        u1, u2 = max(self.uniform(), 1e-300), self.uniform()
        r = math.sqrt(-2.0 * math.log(u1))
        self._spare = r * math.sin(2 * math.pi * u2)
        return mean + std * r * math.cos(2 * math.pi * u2)

    def randint(self, lo: int, hi: int) -> int:
        """Uniform integer in [lo, hi)."""
        return lo + self.gen.next_u64() % max(1, hi - lo)

    def bernoulli(self, p: float = 0.5) -> bool:
        return self.uniform() < p

    def shuffle(self, xs: list) -> list:
        for i in range(len(xs) - 1, 0, -1):
            j = self.randint(0, i + 1)
            xs[i], xs[j] = xs[j], xs[i]
        return xs

    def permutation(self, n: int) -> list:
        return self.shuffle(list(range(n)))

    def choice_k(self, n: int, k: int) -> list:
        return self.permutation(n)[:k]

    def weighted_choice(self, weights) -> int:
        tot = float(sum(weights))
        r, acc = self.uniform() * tot, 0.0
        for i, w in enumerate(weights):
            acc += w
            if r < acc:
                return i
        return len(weights) - 1


@dataclass
class SeedBundle:
    base: int = 0
    data: int = 0
    init: int = 0
    dropout: int = 0
    aug: int = 0

    def to_list(self):
        return [self.base, self.data, self.init, self.dropout, self.aug]


def seed_all(seed: int) -> SeedBundle:
    """Derive per-purpose seeds and seed torch (CPU and CUDA)."""
    import torch

    sm = SplitMix64(seed)
    b = SeedBundle(seed, sm.next_u64(), sm.next_u64(), sm.next_u64(), sm.next_u64())
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    return b


def derived_rngs(seed: int, n: int) -> list:
    sm = SplitMix64(seed)
    return [RNG(sm.next_u64()) for _ in range(n)]


# ---- seed-in, value-out helpers (legacy/src/momijo/learn/utils/randomness.mojo:404-452): each builds a
# fresh generator from ``seed`` (negative seeds use their magnitude), so the same call always returns the
# same value and no global state is touched.
def rng_from_seed(seed: int) -> RNG:
    return RNG(-seed if seed < 0 else seed)


def randint(seed: int, low: int, high: int) -> int:
    return rng_from_seed(seed).randint(low, high)


def uniform(seed: int, low: float = 0.0, high: float = 1.0) -> float:
    return rng_from_seed(seed).uniform(low, high)


def normal(seed: int, mean: float = 0.0, std: float = 1.0) -> float:
    return rng_from_seed(seed).normal(mean, std)


def bernoulli(seed: int, p: float) -> int:
    return int(rng_from_seed(seed).bernoulli(p))


def permutation(seed: int, n: int) -> list:
    return rng_from_seed(seed).permutation(n)


def choice_k(seed: int, n: int, k: int) -> list:
    return rng_from_seed(seed).choice_k(n, k)
