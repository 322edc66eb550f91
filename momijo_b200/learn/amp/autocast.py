"""Mixed-precision policy objects and the gradient scaler
(legacy/src/momijo/learn/amp/autocast.mojo:34-248).

``GradScaler.step(optimizer, found_inf)`` takes ``found_inf`` as an input like the reference;
``check_overflow(grads)`` produces it with the squared-norm / non-finite kernel.
"""
from __future__ import annotations

import contextlib

import torch

from ... import ops


class AMPPrecision:
    FP32, FP16, BF16 = 0, 1, 2
    _names = {0: "fp32", 1: "fp16", 2: "bf16"}

    def __init__(self, code: int = 0):
        self.code = code

    @staticmethod
    def fp32():
        return AMPPrecision(0)

    @staticmethod
    def fp16():
        return AMPPrecision(1)

    @staticmethod
    def bf16():
        return AMPPrecision(2)

    def torch_dtype(self):
        return {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[self.code]

    def __str__(self):
        return self._names[self.code]

    def __eq__(self, o):
        return isinstance(o, AMPPrecision) and o.code == self.code


_STATE = {"enabled": False, "precision": AMPPrecision.fp32()}


class autocast:
    """Flag holder usable as a context manager; layers built on ``momijo_b200.ops`` read it
    through ``autocast.dtype()`` to pick their compute dtype."""

    def __init__(self, enabled: bool = True, precision: AMPPrecision | None = None):
        self.enabled = enabled
        self.precision = precision or AMPPrecision.bf16()
        self._prev = None

    def __enter__(self):
        self._prev = dict(_STATE)
        _STATE.update(enabled=self.enabled, precision=self.precision)
        return self

    def __exit__(self, *exc):
        _STATE.update(self._prev)
        return False

    class _EnabledQuery:
        """``autocast.is_enabled()`` on the class reads the active (context-manager) state; on an instance it
        reads that instance's flag, like the reference's method (legacy/src/momijo/learn/amp/autocast.mojo:88-89)."""

        def __get__(self, obj, owner):
            if obj is None:
                return lambda: _STATE["enabled"]
            return lambda: obj.enabled

    is_enabled = _EnabledQuery()

    # chainable configuration (autocast.mojo:76-92)
    def enable(self) -> "autocast":
        self.enabled = True
        return self

    def disable(self) -> "autocast":
        self.enabled = False
        return self

    def set_precision(self, p: AMPPrecision) -> "autocast":
        self.precision = p
        return self

    def get_precision(self) -> AMPPrecision:
        return self.precision

    def __str__(self):
        return f"autocast(enabled={'true' if self.enabled else 'false'}, precision={self.precision})"

    @staticmethod
    def dtype():
        return _STATE["precision"].torch_dtype() if _STATE["enabled"] else torch.float32


AutocastGuard = autocast


class GradScaler:
    def __init__(self, enabled=True, init_scale=65536.0, growth_factor=2.0, backoff_factor=0.5,
                 growth_interval=2000, min_scale=1.0, max_scale=2.0 ** 64):
        self.enabled = enabled
        self.scale_value = float(init_scale) if enabled else 1.0
        self.init_scale = float(init_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.min_scale, self.max_scale = growth_interval, min_scale, max_scale
        self.growth_tracker = 0

    def get_scale(self) -> float:
        return self.scale_value

    def is_enabled(self) -> bool:
        return self.enabled

    def scale(self, x):
        return x * self.scale_value if self.enabled else x

    def unscale(self, x):
        return x / self.scale_value if self.enabled else x

    def check_overflow(self, grads) -> bool:
        """True if any gradient holds inf/nan (device reduction, one host read)."""
        grads = [g for g in grads if g is not None]
        if not grads:
            return False
        flag = torch.zeros(1, dtype=torch.int32, device=grads[0].device)
        for g in grads:
            if g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous():
                ops.sq_norm(g.reshape(-1), found_inf=flag)
            elif not torch.isfinite(g).all():
                flag.fill_(1)
        return bool(flag.item())

    def step(self, optimizer, found_inf: bool = False) -> bool:
        """Skip the optimizer step on overflow; returns True when the step ran."""
        if self.enabled and found_inf:
            return False
        optimizer.step()
        return True

    def update(self, found_inf: bool = False):
        if not self.enabled:
            return
        if found_inf:
            self.scale_value *= self.backoff_factor
            self.growth_tracker = 0
        else:
            self.growth_tracker += 1
            if self.growth_tracker >= self.growth_interval:
                self.scale_value *= self.growth_factor
                self.growth_tracker = 0
        self.clamp_scale()

    def step_and_update(self, optimizer, found_inf: bool = False, zero_grad_after: bool = True) -> bool:
        ran = self.step(optimizer, found_inf)
        self.update(found_inf)
        if zero_grad_after and hasattr(optimizer, "zero_grad"):
            optimizer.zero_grad()
        return ran

    def clamp_scale(self):
        self.scale_value = min(max(self.scale_value, self.min_scale), self.max_scale)

    def reset(self):
        self.scale_value = self.init_scale if self.enabled else 1.0
        self.growth_tracker = 0

    def state_dict(self):
        return {"scale": self.scale_value, "growth_tracker": self.growth_tracker}

    def load_state_dict(self, d):
        self.scale_value = float(d["scale"])
        self.growth_tracker = int(d["growth_tracker"])
