"""Bitwise image ops with an optional mask (legacy/src/momijo/vision/transforms/bitwise.mojo:27-190)."""
from __future__ import annotations

import torch

from ..image import Image
from .. import kernels as K


def _masked(res: torch.Tensor, mask: Image) -> torch.Tensor:
    if mask is None:
        return res
    m = mask.data[..., :1] != 0
    return torch.where(m, res, torch.zeros_like(res))


def bitwise_and(a: Image, b: Image, mask: Image = None) -> Image:
    return Image(_masked(K.binary(a.data, b.data, K.OP_AND), mask), a.meta().copy())


def bitwise_or(a: Image, b: Image, mask: Image = None) -> Image:
    return Image(_masked(K.binary(a.data, b.data, K.OP_OR), mask), a.meta().copy())


def bitwise_not(a: Image, mask: Image = None) -> Image:
    return Image(_masked(K.binary(a.data, None, K.OP_NOT), mask), a.meta().copy())
