"""Thresholding (legacy/src/momijo/vision/transforms/threshold.mojo:13-48 are shape-only stubs that
never read a pixel; these read them)."""
from __future__ import annotations

import numpy as np
import torch

from ..image import Image
from .. import kernels as K


def _gray(img: Image) -> torch.Tensor:
    d = img.ensure_packed_hwc_u8().data
    return d if d.shape[2] == 1 else K.to_gray(d, bgr=True)


def threshold_binary(img: Image, th: int, maxval: int = 255) -> Image:
    lut = np.where(np.arange(256) > int(th), int(maxval) & 255, 0).astype(np.uint8)
    return Image(K.apply_lut(img.ensure_packed_hwc_u8().data, lut), img.meta().copy())


def otsu_level(hist) -> int:
    hist = np.asarray(hist, dtype=np.float64)
    total = hist.sum()
    if total == 0:
        return 0
    w0 = np.cumsum(hist)
    m = np.cumsum(hist * np.arange(256))
    w1 = total - w0
    valid = (w0 > 0) & (w1 > 0)
    mu0 = np.where(valid, m / np.maximum(w0, 1), 0)
    mu1 = np.where(valid, (m[-1] - m) / np.maximum(w1, 1), 0)
    var = np.where(valid, w0 * w1 * (mu0 - mu1) ** 2, -1.0)
    return int(np.argmax(var))


def threshold_otsu(img: Image, maxval: int = 255) -> Image:
    g = _gray(img)
    t = otsu_level(K.histogram(g, 0).cpu().numpy())
    lut = np.where(np.arange(256) > t, int(maxval) & 255, 0).astype(np.uint8)
    return Image(K.apply_lut(g, lut), img.meta().copy())


def adaptive_threshold(img: Image, maxval=255, method: int = 0, block_size: int = 11, C: int = 2) -> Image:
    """Pixel > (local gaussian mean - C) -> maxval. ``adaptive_threshold(img, method, block, C)`` (the
    reference's first overload) is recognised when ``maxval`` is 0 or 1 and ``method`` looks like a block size."""
    if maxval in (0, 1) and method >= 3:
        maxval, method, block_size, C = 255, maxval, method, block_size
    b = max(int(block_size) | 1, 3)
    g = _gray(img)
    mean = K.gaussian_blur(g, b, b, 0.0).to(torch.int16)
    out = torch.where(g.to(torch.int16) > mean - int(C), int(maxval) & 255, 0).to(torch.uint8)
    return Image(out, img.meta().copy())
