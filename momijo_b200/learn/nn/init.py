"""Weight initialisers: fan computation, gains, Kaiming / Xavier bounds and fills, and the reference's
``SimpleLCG`` bootstrap generator (legacy/src/momijo/learn/nn/init.mojo:48-310).

The ``*_bounds`` / ``*_std`` / ``*_fill`` / ``*_fill_tensor`` functions carry the reference's names and
produce the same numbers for the same generator state (64-bit LCG, uniforms from the top 53 bits,
normals as the sum of twelve uniforms minus six). The ``*_`` functions below them are in-place fills in
the usual torch style, drawing from torch's generator (device tensors included)."""
import math

import torch

_MASK64 = (1 << 64) - 1


class SimpleLCG:
    """state <- 6364136223846793005 * state + 1 (mod 2^64) (legacy/src/momijo/learn/nn/init.mojo:144-176)."""

    def __init__(self, seed: int = 88172645463393265):
        self.state = int(seed) & _MASK64

    def _next_u64(self) -> int:
        self.state = (6364136223846793005 * self.state + 1) & _MASK64
        return self.state

    def rand01(self) -> float:
        return (self._next_u64() >> 11) / 9007199254740992.0   # top 53 bits / 2**53

    def uniform(self, low: float = 0.0, high: float = 1.0) -> float:
        return low + (high - low) * self.rand01()

    def normal01(self) -> float:
        s = 0.0
        for _ in range(12):
            s += self.rand01()
        return s - 6.0

    def normal(self, mean: float = 0.0, std: float = 1.0) -> float:
        return mean + std * self.normal01()


def compute_fan_in_out(shape):
    """(fan_in, fan_out): () -> (1, 1); (n,) -> (n, n); (out, in, *receptive) otherwise."""
    shape = [int(s) for s in shape]
    if len(shape) == 0:
        return 1, 1
    if len(shape) == 1:
        return shape[0], shape[0]
    rf = 1
    for s in shape[2:]:
        rf *= s
    return shape[1] * rf, shape[0] * rf


def calculate_fan_in_and_fan_out(shape):
    if len(shape) < 2:
        raise ValueError("fan in/out need at least 2 dims")
    return compute_fan_in_out(shape)


def calculate_gain(nonlinearity: str, param: float = 0.0) -> float:
    """Unknown names give 1.0, as in the reference (legacy/src/momijo/learn/nn/init.mojo:66-84)."""
    if nonlinearity == "tanh":
        return 5.0 / 3.0
    if nonlinearity == "relu":
        return math.sqrt(2.0)
    if nonlinearity == "leaky_relu":
        return math.sqrt(2.0 / (1.0 + param * param))
    if nonlinearity == "selu":
        return 0.75
    return 1.0


def kaiming_uniform_bounds(shape, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu"):
    fan_in, fan_out = compute_fan_in_out(shape)
    fan = fan_out if mode == "fan_out" else fan_in
    denom = float(fan) if fan > 0 else 1.0
    bound = math.sqrt(3.0) * calculate_gain(nonlinearity, a) / math.sqrt(denom)
    return -bound, bound


def kaiming_normal_std(shape, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu") -> float:
    fan_in, fan_out = compute_fan_in_out(shape)
    fan = fan_out if mode == "fan_out" else fan_in
    denom = float(fan) if fan > 0 else 1.0
    return calculate_gain(nonlinearity, a) / math.sqrt(denom)


def xavier_uniform_bounds(shape, gain: float = 1.0):
    fan_in, fan_out = compute_fan_in_out(shape)
    denom = float(fan_in + fan_out) if fan_in + fan_out > 0 else 1.0
    bound = gain * math.sqrt(6.0 / denom)
    return -bound, bound


def xavier_normal_std(shape, gain: float = 1.0) -> float:
    fan_in, fan_out = compute_fan_in_out(shape)
    denom = float(fan_in + fan_out) if fan_in + fan_out > 0 else 1.0
    return gain * math.sqrt(2.0 / denom)


# ---- list fills (in place; the list's length decides how many values are drawn) ----------------
def _fill_uniform(arr, low, high, rng):
    for i in range(len(arr)):
        arr[i] = rng.uniform(low, high)
    return arr


def _fill_normal(arr, mean, std, rng):
    for i in range(len(arr)):
        arr[i] = rng.normal(mean, std)
    return arr


def kaiming_uniform_fill(arr, shape, a=0.0, mode="fan_in", nonlinearity="leaky_relu", rng=None):
    low, high = kaiming_uniform_bounds(shape, a, mode, nonlinearity)
    return _fill_uniform(arr, low, high, rng or SimpleLCG())


def xavier_uniform_fill(arr, shape, gain=1.0, rng=None):
    low, high = xavier_uniform_bounds(shape, gain)
    return _fill_uniform(arr, low, high, rng or SimpleLCG())


def kaiming_normal_fill(arr, shape, a=0.0, mode="fan_in", nonlinearity="leaky_relu", mean=0.0, rng=None):
    return _fill_normal(arr, mean, kaiming_normal_std(shape, a, mode, nonlinearity), rng or SimpleLCG())


def xavier_normal_fill(arr, shape, gain=1.0, mean=0.0, rng=None):
    return _fill_normal(arr, mean, xavier_normal_std(shape, gain), rng or SimpleLCG())


# ---- tensor fills with the reference generator (row-major order) --------------------------------
def _fill_tensor(t, draw):
    raw = t
    if not isinstance(raw, torch.Tensor):
        from ...tensor.tensor import _raw as unwrap
        raw = unwrap(t)
    n = max(1, raw.numel())
    vals = torch.tensor([draw() for _ in range(n)], dtype=torch.float64)
    with torch.no_grad():
        raw.copy_(vals[: raw.numel()].reshape(raw.shape).to(device=raw.device, dtype=raw.dtype))
    return t


def kaiming_uniform_fill_tensor(t, a=0.0, mode="fan_in", nonlinearity="leaky_relu", rng=None):
    rng = rng or SimpleLCG()
    low, high = kaiming_uniform_bounds(list(t.shape), a, mode, nonlinearity)
    return _fill_tensor(t, lambda: rng.uniform(low, high))


def xavier_uniform_fill_tensor(t, gain=1.0, rng=None):
    rng = rng or SimpleLCG()
    low, high = xavier_uniform_bounds(list(t.shape), gain)
    return _fill_tensor(t, lambda: rng.uniform(low, high))


def kaiming_normal_fill_tensor(t, a=0.0, mode="fan_in", nonlinearity="leaky_relu", mean=0.0, rng=None):
    rng = rng or SimpleLCG()
    std = kaiming_normal_std(list(t.shape), a, mode, nonlinearity)
    return _fill_tensor(t, lambda: rng.normal(mean, std))


def xavier_normal_fill_tensor(t, gain=1.0, mean=0.0, rng=None):
    rng = rng or SimpleLCG()
    std = xavier_normal_std(list(t.shape), gain)
    return _fill_tensor(t, lambda: rng.normal(mean, std))


# ---- torch-style in-place fills ------------------------------------------------------------------
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
    low, high = xavier_uniform_bounds(list(t.shape), gain)
    return uniform_(t, low, high, seed)


def xavier_normal_(t, gain=1.0, seed=None):
    return normal_(t, 0.0, xavier_normal_std(list(t.shape), gain), seed)


def kaiming_uniform_(t, a=0.0, mode="fan_in", nonlinearity="leaky_relu", seed=None):
    low, high = kaiming_uniform_bounds(list(t.shape), a, mode, nonlinearity)
    return uniform_(t, low, high, seed)


def kaiming_normal_(t, a=0.0, mode="fan_in", nonlinearity="leaky_relu", seed=None):
    return normal_(t, 0.0, kaiming_normal_std(list(t.shape), a, mode, nonlinearity), seed)
