"""Factories (legacy/src/momijo/tensor/creation.mojo:57-1509): typed zeros/ones/full/eye/arange/
linspace/rand/randn/randperm/from_list families. Every random factory takes an explicit seed and
the same seed gives the same values (``SplitMix64`` / ``RNG64`` in the reference; torch's seeded
generator here)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .tensor import Tensor, _wrap

_F32, _F64, _I64, _I32, _I16, _I8, _U8, _B = (torch.float32, torch.float64, torch.int64, torch.int32,
                                            torch.int16, torch.int8, torch.uint8, torch.bool)


class SplitMix64:
    def __init__(self, seed: int = 0):
        self.state = seed & ((1 << 64) - 1)

    def next_u64(self) -> int:
        M = (1 << 64) - 1
        self.state = (self.state + 0x9E3779B97F4A7C15) & M
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    next = next_u64


class RNG64(SplitMix64):
    """SplitMix64 stream with float and bounded-integer draws (legacy/src/momijo/tensor/creation.mojo:78-126)."""

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)

    next_f64 = uniform

    def next_f32(self) -> float:
        return float(torch.tensor(self.uniform(), dtype=torch.float32))

    def next_i32(self, low: int, high: int) -> int:
        """Unbiased integer in [low, high): draws above the largest multiple of the span are rejected."""
        span = high - low
        if span <= 0:
            return low
        full = 0xFFFFFFFFFFFFFFFF
        limit = full - (full % span)
        u = self.next_u64()
        while u >= limit:
            u = self.next_u64()
        return low + u % span


def _shape(shape):
    return [shape] if isinstance(shape, int) else list(shape)


def _dev(ctx):
    """``ctx`` may be a RuntimeDeviceContext / Device / torch device / None."""
    if ctx is None:
        return None
    if hasattr(ctx, "torch_device"):
        return ctx.torch_device()
    return ctx


def _gen(seed):
    return torch.Generator().manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)


def zeros(shape, dtype=_F64, ctx=None):
    return _wrap(torch.zeros(_shape(shape), dtype=dtype, device=_dev(ctx)))


def ones(shape, dtype=_F64, ctx=None):
    return _wrap(torch.ones(_shape(shape), dtype=dtype, device=_dev(ctx)))


def full(shape, value, dtype=None, ctx=None):
    return _wrap(torch.full(_shape(shape), value, dtype=dtype, device=_dev(ctx)))


def empty(shape, dtype=_F64, ctx=None):
    return _wrap(torch.empty(_shape(shape), dtype=dtype, device=_dev(ctx)))


def zeros_like(x):
    return _wrap(torch.zeros_like(x))


def ones_like(x):
    return _wrap(torch.ones_like(x))


def full_like(x, v):
    return _wrap(torch.full_like(x, v))


def eye(n, m=None, dtype=_F64):
    return _wrap(torch.eye(n, m if m is not None else n, dtype=dtype))


def scalar_f64(v):
    return _wrap(torch.tensor(float(v), dtype=_F64))


def scalar_f32(v):
    return _wrap(torch.tensor(float(v), dtype=_F32))


def scalar_int(v):
    return _wrap(torch.tensor(int(v), dtype=_I64))


def _typed(fn_name, fn, table):
    for suffix, dt in table.items():
        def f(*a, _dt=dt, **k):
            return fn(*a, dtype=_dt, **k)
        f.__name__ = f"{fn_name}_{suffix}"
        globals()[f.__name__] = f


_T = {"f64": _F64, "f32": _F32, "int": _I64, "i32": _I32, "i16": _I16, "i8": _I8, "u8": _U8, "bool": _B}
_typed("zeros", zeros, _T)
_typed("ones", ones, _T)
_typed("empty", empty, _T)
_typed("eye", eye, {"f64": _F64, "f32": _F32, "int": _I64})


def arange_dt(start, stop=None, step=1, dtype=_F64):
    if stop is None:
        start, stop = 0, start
    return _wrap(torch.arange(start, stop, step, dtype=dtype))


def arange_f64(start, stop=None, step=1):
    return arange_dt(start, stop, step, _F64)


def arange_f32(start, stop=None, step=1):
    return arange_dt(start, stop, step, _F32)


def arange_int(start, stop=None, step=1):
    return arange_dt(start, stop, step, _I64)


arange = arange_f32


def linspace_f64(start, stop, num, endpoint=True):
    if not endpoint and num > 0:
        stop = start + (stop - start) * (num - 1) / num
    return _wrap(torch.linspace(start, stop, num, dtype=_F64))


def linspace_f32(start, stop, num, endpoint=True):
    return _wrap(linspace_f64(start, stop, num, endpoint).to(_F32))


def linspace_int(start, stop, num, endpoint=True):
    return _wrap(linspace_f64(start, stop, num, endpoint).round().to(_I64))


def rand(shape, seed=0, dtype=_F64, seed_ref=None):
    """``rand(shape, seed, dtype)``; the reference's ``rand(x, low, high, seed)`` (legacy/src/momijo/tensor/
    creation.mojo:708-711) draws uniform values in [low, high) with the shape of tensor ``x``."""
    if isinstance(shape, torch.Tensor):
        low, high = float(seed), float(dtype) if not isinstance(dtype, torch.dtype) else 1.0
        u = torch.rand(list(shape.shape), generator=_gen(seed_ref or 0), dtype=torch.float64)
        return _wrap((low + (high - low) * u).to(shape.dtype if shape.dtype.is_floating_point else torch.float64))
    return _wrap(torch.rand(_shape(shape), generator=_gen(seed), dtype=torch.float64).to(dtype))


def randn(shape, seed: int = 0, dtype=_F64):
    return _wrap(torch.randn(_shape(shape), generator=_gen(seed), dtype=torch.float64).to(dtype))


def randn_f64(shape, seed: int = 0):
    return randn(shape, seed, _F64)


def randn_f32(shape, seed: int = 0):
    return randn(shape, seed, _F32)


def randn_int(shape, seed: int = 0):
    return _wrap(randn(shape, seed, _F64).round().to(_I64))


def rand_f64(shape, seed: int = 0):
    return rand(shape, seed, _F64)


def rand_f32(shape, seed: int = 0):
    return rand(shape, seed, _F32)


def normal(shape, mean=0.0, std=1.0, seed: int = 0, dtype=_F64):
    return _wrap((randn(shape, seed, _F64) * std + mean).to(dtype))


def uniform(shape, lo=0.0, hi=1.0, seed: int = 0, dtype=_F64):
    return _wrap((rand(shape, seed, _F64) * (hi - lo) + lo).to(dtype))


def randint(shape, lo, hi, seed: int = 0):
    return _wrap(torch.randint(lo, hi, _shape(shape), generator=_gen(seed)))


def bernoulli(shape, p=0.5, seed: int = 0):
    return _wrap((torch.rand(_shape(shape), generator=_gen(seed)) < p).to(_I64))


bernoulli_int = bernoulli


def bernoulli_f64(shape, p=0.5, seed: int = 0):
    return _wrap(bernoulli(shape, p, seed).to(_F64))


def randperm_int(n, seed: int = 0):
    return _wrap(torch.randperm(n, generator=_gen(seed)))


def randperm_f64(n, seed: int = 0):
    return _wrap(randperm_int(n, seed).to(_F64))


def randperm_f32(n, seed: int = 0):
    return _wrap(randperm_int(n, seed).to(_F32))


def _from_list(dt):
    def f(xs, shape: Optional[Sequence[int]] = None):
        t = torch.tensor(xs, dtype=dt)
        return _wrap(t.reshape(list(shape)) if shape is not None else t)
    return f


for _name, _dt in {"float64": _F64, "float32": _F32, "int": _I64, "int32": _I32, "int16": _I16,
                   "int8": _I8, "uint8": _U8, "bool": _B}.items():
    globals()[f"from_list_{_name}"] = _from_list(_dt)
    globals()[f"from_2d_list_{_name}"] = _from_list(_dt)
    globals()[f"from_3d_list_{_name}"] = _from_list(_dt)


def from_list(xs, dtype=None, shape=None):
    t = torch.tensor(xs, dtype=dtype)
    return _wrap(t.reshape(list(shape)) if shape is not None else t)


# ---- the remaining typed names of the reference (legacy/src/momijo/tensor/creation.mojo:39-1500) -------------------
# One family per dtype suffix, generated from the generic factory; the ``*_with`` forms take the reference's
# element converter (``f``) and apply it to every generated value, so any Python callable works.
_ALL_DT = {"f16": torch.float16, "f32": _F32, "f64": _F64, "i8": _I8, "i16": _I16, "i32": _I32, "i64": _I64,
           "u8": _U8, "u16": torch.uint16, "u32": torch.uint32, "u64": torch.uint64, "int": _I64}


def _cast(t, dt):
    """Cast with wrap-around for the unsigned types that torch cannot reach directly from every source."""
    if dt in (torch.uint16, torch.uint32, torch.uint64):
        return t.to(torch.int64).to(dt)
    return t.to(dt)


def clamp01(x: float) -> float:
    return 0.0 if x < 0.0 else (1.0 if x > 1.0 else x)


def rotl64(x: int, k: int) -> int:
    k &= 63
    x &= (1 << 64) - 1
    return x if k == 0 else ((x << k) | (x >> (64 - k))) & ((1 << 64) - 1)


def init_rng(seed=None) -> RNG64:
    return RNG64(0xD1B54A32D192ED03 if seed is None else int(seed))


def zero_scalar_of(from_f64):
    return from_f64(0.0)


def scalar_zero_tensor(dtype=_F64):
    return _wrap(torch.zeros((), dtype=dtype))


def _apply(t, f):
    if f is None:
        return _wrap(t)
    flat = [f(v) for v in t.reshape(-1).tolist()]
    return _wrap(torch.tensor(flat).reshape(t.shape))


def empty_tensor(dtype=_F64):
    return _wrap(torch.zeros(0, dtype=dtype))


def empty_tensor_with(from_f64=None, shape=None):
    return _apply(torch.zeros(_shape(shape) if shape is not None else [0], dtype=_F64), from_f64)


def empty_like(x):
    from .tensor import _raw
    return _wrap(torch.empty_like(_raw(x)))


def zeros_with_shape(shape, from_f64=None): return _apply(torch.zeros(_shape(shape), dtype=_F64), from_f64)    # noqa: E704
def ones_with_shape(shape, from_f64=None): return _apply(torch.ones(_shape(shape), dtype=_F64), from_f64)      # noqa: E704
def eye_with_shape(rows, cols, from_f64=None): return _apply(torch.eye(rows, cols, dtype=_F64), from_f64)      # noqa: E704


def arange_with(start, f=None, stop=-1, step=1):
    """``arange(start, stop, step)``; with ``stop`` left at -1 the range is ``[0, start)``."""
    if stop == -1:
        start, stop = 0, start
    return _apply(torch.arange(start, stop, step), f)


def linspace_list_f64(a: float, b: float, n: int, endpoint: bool = True):
    if n <= 0:
        return []
    if n == 1:
        return [float(a)]
    step = (b - a) / (n - 1 if endpoint else n)
    return [a + i * step for i in range(n)]


def linspace_with(a, b, n, f=None, endpoint=True):
    return _apply(torch.tensor(linspace_list_f64(a, b, n, endpoint), dtype=_F64), f)


def linspace_Int(a, b, n, endpoint=True):
    return _wrap(torch.tensor([int(v) for v in linspace_list_f64(a, b, n, endpoint)], dtype=_I64))


def randu_with(shape, f=None, low=0.0, high=1.0, seed=None):
    t = torch.rand(_shape(shape), generator=_gen(0 if seed is None else seed), dtype=_F64) * (high - low) + low
    return _apply(t, f)


rand_with_shape = randu_with


def rand_like_with(x, f=None, low=0.0, high=1.0, seed=None):
    return randu_with(list(x.shape), f, low, high, seed)


def bernoulli_with(shape, p, f=None, seed=None):
    t = (torch.rand(_shape(shape), generator=_gen(0 if seed is None else seed), dtype=_F64) < p).to(_I64)
    return _apply(t, f)


def randperm_with(n, f=None, seed=None):
    return _apply(torch.randperm(n, generator=_gen(0 if seed is None else seed)), f)


def normal_f32(shape, mean=0.0, std=1.0, seed: int = 0):
    return normal(shape, mean, std, seed, _F32)


def from_2d_list(xs, dtype=None):
    return from_list(xs, dtype)


def from_3d_list(xs, dtype=None):
    return from_list(xs, dtype)


def _u01(shape, seed):
    return torch.rand(_shape(shape), generator=_gen(0 if seed is None else seed), dtype=_F64)


def _mk_typed():
    g = globals()

    def family(dt):
        wide = _F64 if dt.is_floating_point else _I64

        def arange_(start, stop=None, step=1):
            lo, hi = (0, start) if stop is None else (start, stop)
            return _wrap(_cast(torch.arange(lo, hi, step, dtype=wide), dt))

        def bernoulli_(shape, p=0.5, seed=0):
            return _wrap(_cast((_u01(shape, seed) < p).to(_I64), dt))

        def randperm_(n, seed=0):
            return _wrap(_cast(torch.randperm(n, generator=_gen(seed)), dt))

        def randu_(shape, low=0.0, high=1.0, seed=None):
            return _wrap(_cast(_u01(shape, seed) * (high - low) + low, dt))

        def rand_like_(x, low=0.0, high=1.0, seed=None):
            return randu_(list(x.shape), low, high, seed)

        def randn_like_(x, seed=0):
            return _wrap(_cast(torch.randn(list(x.shape), generator=_gen(seed), dtype=_F64), dt))

        return {"arange": arange_, "bernoulli": bernoulli_, "randperm": randperm_, "randu": randu_,
                "rand_like": rand_like_, "randn_like": randn_like_}

    for sfx, dt in _ALL_DT.items():
        for base, fn in family(dt).items():
            g.setdefault(f"{base}_{sfx}", fn)
    for base in ("arange", "bernoulli", "rand_like", "randn_like"):
        for sfx in ("f32", "f64", "int"):
            g.setdefault(f"{base}_{sfx}_alias", g[f"{base}_{sfx}"])


_mk_typed()
