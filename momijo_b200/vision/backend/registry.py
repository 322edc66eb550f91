"""Kernel registry (legacy/src/momijo/vision/backend/registry.mojo:25-56). The reference picks between
``CPUScalar`` and ``CPUSIMD`` loops; here the choice is between the host restatement and the CUDA kernels,
made per call from where the image lives, and the registry lets a caller pin one or swap a kernel in."""
from __future__ import annotations

from enum import IntEnum
from typing import Callable, Dict

import torch

from .. import kernels as K
from .schedule import Schedule, default_schedule


class BackendKind(IntEnum):
    CPUScalar = 0
    CPUSIMD = 1
    CUDA = 2


Backend = BackendKind   # the reference's name for the enumeration (registry.mojo:25-27)


class KernelRegistry:
    def __init__(self, kind: BackendKind = None, schedule: Schedule = None):
        if kind is None:
            kind = BackendKind.CUDA if torch.cuda.is_available() else BackendKind.CPUSIMD
        self._kind = BackendKind(kind)
        self._schedule = schedule or default_schedule()
        self._table: Dict[str, Callable] = {
            "resize_nearest": lambda t, oh, ow: K.resize(t, oh, ow, False),
            "resize_bilinear": lambda t, oh, ow: K.resize(t, oh, ow, True),
            "rgb_to_gray": lambda t: K.to_gray(t, False),
            "swap_rb": K.swap_rb,
            "gaussian": lambda t, k: K.gaussian_blur(t, k, k, 0.0),
            "erode": lambda t, k: K.morph(t, k, False),
            "dilate": lambda t, k: K.morph(t, k, True),
        }

    def kind(self) -> BackendKind:
        return self._kind

    def with_auto(self) -> "KernelRegistry":
        """The same backend with the automatic schedule for an unknown image size
        (legacy/src/momijo/vision/backend/registry.mojo:37-39)."""
        from .schedule import auto_schedule
        return KernelRegistry(self._kind, auto_schedule(0, 0))

    def schedule(self) -> Schedule:
        return self._schedule

    def set_schedule(self, s: Schedule):
        self._schedule = s

    def register(self, name: str, fn: Callable):
        self._table[name] = fn

    def has(self, name: str) -> bool:
        return name in self._table

    def place(self, t: torch.Tensor) -> torch.Tensor:
        """Move an image to the memory this registry's kernels run in."""
        if self._kind == BackendKind.CUDA:
            return t if t.is_cuda else t.cuda()
        return t.cpu() if t.is_cuda else t

    def run(self, name: str, t: torch.Tensor, *args) -> torch.Tensor:
        return self._table[name](self.place(t), *args)

    # names used by code written against the reference
    def resize_nearest(self, t, oh, ow):
        return self.run("resize_nearest", t, oh, ow)

    def convert_rgb_to_gray(self, t):
        return self.run("rgb_to_gray", t)


def default_registry() -> KernelRegistry:
    return KernelRegistry()
