"""The vision package's own small tensor type is a strided raw pointer in the reference
(legacy/src/momijo/vision/tensor.mojo:35); here it is a torch tensor, and this module keeps the
helper names that code written against the reference imports."""
from __future__ import annotations

import torch

Tensor = torch.Tensor


def packed_hwc_strides(h: int, w: int, c: int):
    return (w * c, c, 1)


def packed_chw_strides(c: int, h: int, w: int):
    return (h * w, w, 1)
