"""Learning-rate schedulers with ``get_lr / step / step_to / state_dict / load_state_dict``
(legacy/src/momijo/learn/optim/schedulers.mojo:91-1197). ``last_epoch`` starts at -1; ``step()``
increments it, then computes; negative epochs return ``base_lr``. State dicts are the
single-quoted pseudo-JSON strings of the reference (schedulers.mojo:254-260). Exact ``cos`` /
``pow`` replace the reference's series approximations."""
from __future__ import annotations

import ast
import math


class _Scheduler:
    _fields = ()

    def __init__(self):
        self.last_epoch = -1

    def lr_at(self, t: int) -> float:
        raise NotImplementedError

    def get_lr(self) -> float:
        return self.base_lr if self.last_epoch < 0 else self.lr_at(self.last_epoch)

    def step(self) -> float:
        self.last_epoch += 1
        return self.get_lr()

    def step_to(self, epoch: int) -> float:
        self.last_epoch = epoch
        return self.get_lr()

    def state_dict(self) -> str:
        items = [("type", type(self).__name__)] + [(f, getattr(self, f)) for f in self._fields]
        items.append(("last_epoch", self.last_epoch))
        return "{" + ",".join(f"'{k}':{v!r}" for k, v in items) + "}"

    def load_state_dict(self, s) -> bool:
        try:
            d = ast.literal_eval(s) if isinstance(s, str) else dict(s)
        except Exception:
            return False
        for k, v in d.items():
            if k != "type" and hasattr(self, k):
                setattr(self, k, v)
        return True


class StepLR(_Scheduler):
    _fields = ("base_lr", "step_size", "gamma")

    def __init__(self, base_lr, step_size, gamma=0.1):
        super().__init__()
        self.base_lr, self.step_size, self.gamma = base_lr, step_size, gamma

    def lr_at(self, t):
        return self.base_lr * self.gamma ** (t // self.step_size)


class ExponentialLR(_Scheduler):
    _fields = ("base_lr", "gamma")

    def __init__(self, base_lr, gamma=0.99):
        super().__init__()
        self.base_lr, self.gamma = base_lr, gamma

    def lr_at(self, t):
        return self.base_lr * self.gamma ** t


class MultiStepLR(_Scheduler):
    _fields = ("base_lr", "milestones", "gamma")

    def __init__(self, base_lr, milestones, gamma=0.1):
        super().__init__()
        self.base_lr, self.milestones, self.gamma = base_lr, sorted(milestones), gamma

    def lr_at(self, t):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if m <= t)


class PolynomialLR(_Scheduler):
    _fields = ("base_lr", "T_max", "power", "min_lr")

    def __init__(self, base_lr, T_max, power=1.0, min_lr=0.0):
        super().__init__()
        self.base_lr, self.T_max, self.power, self.min_lr = base_lr, T_max, power, min_lr

    def lr_at(self, t):
        f = 1.0 - min(t, self.T_max) / self.T_max
        return self.min_lr + (self.base_lr - self.min_lr) * f ** self.power


class CosineAnnealingLR(_Scheduler):
    _fields = ("base_lr", "T_max", "min_lr")

    def __init__(self, base_lr, T_max, min_lr=0.0):
        super().__init__()
        self.base_lr, self.T_max, self.min_lr = base_lr, T_max, min_lr

    def lr_at(self, t):
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (
            1.0 + math.cos(math.pi * min(t, self.T_max) / self.T_max))


class CosineAnnealingWarmRestarts(_Scheduler):
    _fields = ("base_lr", "T_0", "T_mult", "min_lr")

    def __init__(self, base_lr, T_0, T_mult=1, min_lr=0.0):
        super().__init__()
        self.base_lr, self.T_0, self.T_mult, self.min_lr = base_lr, T_0, T_mult, min_lr

    def _cycle(self, t):
        Ti, start = self.T_0, 0
        while t >= start + Ti:
            start += Ti
            Ti *= self.T_mult
        return t - start, Ti

    def lr_at(self, t):
        tc, Ti = self._cycle(t)
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1.0 + math.cos(math.pi * tc / Ti))


class LinearWarmup(_Scheduler):
    _fields = ("start_lr", "base_lr", "warmup_steps")

    def __init__(self, start_lr, base_lr, warmup_steps):
        super().__init__()
        self.start_lr, self.base_lr, self.warmup_steps = start_lr, base_lr, warmup_steps

    def get_lr(self):
        return self.start_lr if self.last_epoch < 0 else self.lr_at(self.last_epoch)

    def lr_at(self, t):
        if t >= self.warmup_steps:
            return self.base_lr
        return self.start_lr + (self.base_lr - self.start_lr) * t / self.warmup_steps


class WarmupThen(_Scheduler):
    """Warm up for ``warmup.warmup_steps`` steps, then ``main.step_to(t - warmup_steps)``."""

    def __init__(self, warmup: LinearWarmup, main: _Scheduler):
        super().__init__()
        self.warmup, self.main = warmup, main
        self.base_lr = warmup.start_lr

    def lr_at(self, t):
        w = self.warmup.warmup_steps
        return self.warmup.lr_at(t) if t < w else self.main.step_to(t - w)

    def state_dict(self):
        return "{'type':'WarmupThen','last_epoch':%d,'warmup':%s,'main':%s}" % (
            self.last_epoch, self.warmup.state_dict(), self.main.state_dict())

    def load_state_dict(self, s):
        try:
            d = ast.literal_eval(s) if isinstance(s, str) else dict(s)
        except Exception:
            return False
        self.last_epoch = d.get("last_epoch", self.last_epoch)
        self.warmup.load_state_dict(d.get("warmup", {}))
        self.main.load_state_dict(d.get("main", {}))
        return True


class ChainedLR(_Scheduler):
    """Piecewise: scheduler k runs over ``spans[k]`` steps (the last one runs on)."""

    def __init__(self, schedulers, spans):
        super().__init__()
        self.schedulers, self.spans = list(schedulers), list(spans)
        self.base_lr = self.schedulers[0].base_lr if hasattr(self.schedulers[0], "base_lr") else 0.0

    def lr_at(self, t):
        start = 0
        for k, (s, span) in enumerate(zip(self.schedulers, self.spans)):
            if t < start + span or k == len(self.schedulers) - 1:
                return s.step_to(t - start)
            start += span
        return self.schedulers[-1].step_to(t - start)

    def state_dict(self):
        return "{'type':'ChainedLR','last_epoch':%d,'spans':%r}" % (self.last_epoch, self.spans)


class ReduceLROnPlateau:
    """Improvement is beyond ``best -/+ threshold`` (absolute); reduce when ``num_bad > patience``
    and not cooling down (schedulers.mojo:1045-1181)."""

    def __init__(self, lr, factor=0.1, patience=10, threshold=1e-4, cooldown=0, min_lr=0.0, mode="min"):
        self.lr, self.factor, self.patience, self.threshold = lr, factor, patience, threshold
        self.cooldown, self.min_lr, self.mode = cooldown, min_lr, mode
        self.best = math.inf if mode == "min" else -math.inf
        self.num_bad, self.cooldown_counter, self.last_epoch = 0, 0, -1

    def get_lr(self):
        return self.lr

    def _improved(self, v):
        return v < self.best - self.threshold if self.mode == "min" else v > self.best + self.threshold

    def step(self, metric: float) -> float:
        self.last_epoch += 1
        if self._improved(metric):
            self.best, self.num_bad = metric, 0
        else:
            self.num_bad += 1
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.num_bad = 0
        if self.num_bad > self.patience:
            self.lr = max(self.lr * self.factor, self.min_lr)
            self.cooldown_counter, self.num_bad = self.cooldown, 0
        return self.lr

    def state_dict(self):
        return ("{'type':'ReduceLROnPlateau','lr':%r,'best':%r,'num_bad':%d,'cooldown_counter':%d,"
                "'last_epoch':%d}" % (self.lr, self.best, self.num_bad, self.cooldown_counter, self.last_epoch))

    def load_state_dict(self, s):
        try:
            d = ast.literal_eval(s.replace("inf", "1e999")) if isinstance(s, str) else dict(s)
        except Exception:
            return False
        for k, v in d.items():
            if k != "type" and hasattr(self, k):
                setattr(self, k, v)
        return True


# ---- setters of the reference (legacy/src/momijo/learn/optim/schedulers.mojo:126-131, 213-222, 388-404, 535-550,
# 657-669, 781-795, 1111-1150). They clamp like the reference and do not recompute the current rate: the next
# ``step`` / ``step_to`` does. --------------------------------------------------------------------------------------
def _set_base_lr(self, lr: float) -> None:
    self.base_lr = max(float(lr), 0.0, getattr(self, "min_lr", 0.0))


def _set_min_lr(self, lr: float) -> None:
    v = max(float(lr), 0.0)
    if hasattr(self, "base_lr") and self.base_lr < v:
        self.base_lr = v
    self.min_lr = v
    if hasattr(self, "lr") and self.lr < v:
        self.lr = v


def _set_gamma(self, g: float) -> None:
    self.gamma = g if g > 0.0 else 0.99


def _set_power(self, p: float) -> None:
    self.power = max(float(p), 0.0)


def _set_start_lr(self, lr: float) -> None:
    self.start_lr = max(float(lr), 0.0)


def _set_warmup_steps(self, steps: int) -> None:
    self.warmup_steps = steps if steps > 0 else 1


for _cls in (StepLR, ExponentialLR, MultiStepLR, PolynomialLR, CosineAnnealingLR, CosineAnnealingWarmRestarts, LinearWarmup):
    _cls.set_base_lr = _set_base_lr
for _cls in (PolynomialLR, CosineAnnealingLR, CosineAnnealingWarmRestarts, ReduceLROnPlateau):
    _cls.set_min_lr = _set_min_lr
ExponentialLR.set_gamma = StepLR.set_gamma = MultiStepLR.set_gamma = _set_gamma
PolynomialLR.set_power = _set_power
LinearWarmup.set_start_lr, LinearWarmup.set_warmup_steps = _set_start_lr, _set_warmup_steps


def _plateau_set_mode(self, mode: str) -> None:
    """Anything but "max" means "min"; the best value restarts for the new direction."""
    self.mode = "max" if mode == "max" else "min"
    self.best = -math.inf if self.mode == "max" else math.inf


ReduceLROnPlateau.set_mode = _plateau_set_mode
ReduceLROnPlateau.set_factor = lambda self, v: setattr(self, "factor", v if v > 0.0 else 0.1)
ReduceLROnPlateau.set_patience = lambda self, k: setattr(self, "patience", max(int(k), 0))
ReduceLROnPlateau.set_threshold = lambda self, v: setattr(self, "threshold", max(float(v), 0.0))
ReduceLROnPlateau.set_cooldown = lambda self, v: setattr(self, "cooldown", max(int(v), 0))
