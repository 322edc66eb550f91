"""Weight initialisers: fan computation, gains, Kaiming / Xavier fills and the reference's
``SimpleLCG`` generator (legacy/src/momijo/learn/nn/init.mojo:48-294)."""
import math

import torch


class SimpleLCG:
    """32-bit LCG ``state * 1664525 + 1013904223`` yielding uniforms in [0, 1)."""

    def __init__(self, seed: int = 42):
        self.state = seed & 0xFFFFFFFF

    def next_u32(self) -> int:
        self.state = (self.state * 1664525 + 1013904223) & 0xFFFFFFFF
        return self.state

    def uniform(self) -> float:
        return self.next_u32() / 4294967296.0

    def normal(self) -> float:
        u1, u2 = max(self.uniform(), 1e-12), self.uniform()
        return math.sqrt(-2.0 * math.log(u1)) * math.cos(2.0 * math.pi * u2)


def calculate_fan_in_and_fan_out(shape):
    if len(shape) < 2:
        raise ValueError("fan in/out need at least 2 dims")
    rf = 1
    for s in shape[2:]:
        rf *= s
    return shape[1] * rf, shape[0] * rf


def calculate_gain(nonlinearity: str, param: float = 0.01) -> float:
    return {"linear": 1.0, "conv2d": 1.0, "sigmoid": 1.0, "tanh": 5.0 / 3.0,
            "relu": math.sqrt(2.0), "selu": 0.75,
            "leaky_relu": math.sqrt(2.0 / (1 + param ** 2))}[nonlinearity]


def _gen(seed):
    return None if seed is None else torch.Generator().manual_seed(seed)


@torch.no_grad()
def uniform_(t, a=0.0, b=1.0, seed=None):
    return t.copy_(torch.empty(t.shape).uniform_(a, b, generator=_gen(seed)).to(t.dtype))


@torch.no_grad()
def normal_(t, mean=0.0, std=1.0, seed=None):
    return t.copy_(torch.empty(t.shape).normal_(mean, std, generator=_gen(seed)).to(t.dtype))


@torch.no_grad()
def constant_(t, v):
    return t.fill_(v)


def zeros_(t):
    return constant_(t, 0.0)


def ones_(t):
    return constant_(t, 1.0)


def xavier_uniform_(t, gain=1.0, seed=None):
    fi, fo = calculate_fan_in_and_fan_out(t.shape)
    a = gain * math.sqrt(6.0 / (fi + fo))
    return uniform_(t, -a, a, seed)


def xavier_normal_(t, gain=1.0, seed=None):
    fi, fo = calculate_fan_in_and_fan_out(t.shape)
    return normal_(t, 0.0, gain * math.sqrt(2.0 / (fi + fo)), seed)


def kaiming_uniform_(t, a=0.0, mode="fan_in", nonlinearity="leaky_relu", seed=None):
    fi, fo = calculate_fan_in_and_fan_out(t.shape)
    fan = fi if mode == "fan_in" else fo
    bound = calculate_gain(nonlinearity, a) * math.sqrt(3.0 / fan)
    return uniform_(t, -bound, bound, seed)


def kaiming_normal_(t, a=0.0, mode="fan_in", nonlinearity="leaky_relu", seed=None):
    fi, fo = calculate_fan_in_and_fan_out(t.shape)
    fan = fi if mode == "fan_in" else fo
    return normal_(t, 0.0, calculate_gain(nonlinearity, a) / math.sqrt(fan), seed)
