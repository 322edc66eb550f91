"""Augmentation pipeline on float CHW tensors (legacy/src/momijo/vision/transforms/compose.mojo:27-300,
normalize.mojo:16-88, transforms.mojo:26-86)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Sequence

import torch
import torch.nn.functional as F


@dataclass
class StepAffine:
    max_rotate_deg: float = 0.0
    max_translate: float = 0.0
    min_scale: float = 1.0
    max_scale: float = 1.0
    p: float = 1.0


@dataclass
class StepNorm:
    mean: Sequence[float] = (0.0,)
    std: Sequence[float] = (1.0,)


@dataclass
class Step:
    kind: int
    affine: StepAffine = None
    norm: StepNorm = None


def make_step_affine(a: StepAffine) -> Step:
    return Step(0, a, None)


def make_step_norm(nm: StepNorm) -> Step:
    return Step(1, None, nm)


def normalize_chw(x: torch.Tensor, mean: Sequence[float], std: Sequence[float]) -> torch.Tensor:
    c = x.shape[-3]
    m = torch.tensor([mean[min(i, len(mean) - 1)] for i in range(c)], dtype=x.dtype, device=x.device).view(c, 1, 1)
    s = torch.tensor([std[min(i, len(std) - 1)] for i in range(c)], dtype=x.dtype, device=x.device).view(c, 1, 1)
    s = torch.where(s.abs() < 1e-12, torch.ones_like(s), s)
    return (x - m) / s


class Normalize:
    def __init__(self, mean=(0.0, 0.0, 0.0), std=(1.0, 1.0, 1.0)):
        self.mean, self.std = tuple(mean), tuple(std)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return normalize_chw(x, self.mean, self.std)


def normalize(x: torch.Tensor, mean, std) -> torch.Tensor:
    return normalize_chw(x, mean, std)


def to_tensor(img) -> torch.Tensor:
    """HWC uint8 image (or tensor) -> CHW float32 in [0, 1]."""
    from ..image import Image
    d = img.data if isinstance(img, Image) else torch.as_tensor(img)
    if d.dtype == torch.uint8:
        return d.permute(2, 0, 1).to(torch.float32) / 255.0
    return d.to(torch.float32)


def random_affine(x: torch.Tensor, a: StepAffine, gen: torch.Generator = None) -> torch.Tensor:
    r = torch.rand(5, generator=gen).tolist()
    if r[0] >= a.p:
        return x
    ang = math.radians((2 * r[1] - 1) * a.max_rotate_deg)
    sc = a.min_scale + (a.max_scale - a.min_scale) * r[2]
    tx, ty = (2 * r[3] - 1) * a.max_translate, (2 * r[4] - 1) * a.max_translate
    c, s = math.cos(ang) / sc, math.sin(ang) / sc
    theta = torch.tensor([[c, s, tx], [-s, c, ty]], dtype=x.dtype, device=x.device).unsqueeze(0)
    xb = x.unsqueeze(0) if x.dim() == 3 else x
    grid = F.affine_grid(theta.expand(xb.shape[0], -1, -1), list(xb.shape), align_corners=False)
    out = F.grid_sample(xb, grid, mode="bilinear", padding_mode="zeros", align_corners=False)
    return out[0] if x.dim() == 3 else out


class Compose:
    """Ordered list of callables and/or parameterised steps."""

    def __init__(self, fns: List[Callable] = None, seed: int = None):
        self.fns: List = list(fns or [])
        self.gen = torch.Generator()
        if seed is not None:
            self.gen.manual_seed(int(seed))

    def add(self, fn: Callable):
        self.fns.append(fn)
        return self

    def add_random_affine(self, max_rotate_deg=0.0, max_translate=0.0, min_scale=1.0, max_scale=1.0, p=1.0):
        self.fns.append(make_step_affine(StepAffine(max_rotate_deg, max_translate, min_scale, max_scale, p)))
        return self

    def add_normalize(self, mean, std):
        self.fns.append(make_step_norm(StepNorm(list(mean), list(std))))
        return self

    def apply(self, x):
        for f in self.fns:
            if isinstance(f, Step):
                x = random_affine(x, f.affine, self.gen) if f.kind == 0 else normalize_chw(x, f.norm.mean, f.norm.std)
            else:
                x = f(x)
        return x

    __call__ = apply

    def __len__(self):
        return len(self.fns)


def build_transforms(img_size: int = 28, augment: bool = False) -> Compose:
    c = Compose()
    if augment:
        c.add_random_affine(10.0, 0.1, 0.9, 1.1, 0.5)
    c.add_normalize([0.5], [0.5])
    return c
