"""Smoothing and edge filters (legacy/src/momijo/vision/transforms/filter.mojo). ``sobel``,
``laplacian`` and ``canny`` return a copy of the input in the reference (filter.mojo:199-250);
here they compute 3x3 derivatives and a full Canny (non-maximum suppression + hysteresis)."""
from __future__ import annotations

import numpy as np
import torch

from ..image import Image
from .. import kernels as K


def _odd(v: int, lo: int = 1) -> int:
    v = max(int(v), lo)
    return v if v & 1 else v + 1


def _like(img, data):
    return Image(data, img.meta().copy())


def _gray_data(img: Image) -> torch.Tensor:
    d = img.ensure_packed_hwc_u8().data
    return d if d.shape[2] == 1 else K.to_gray(d, bgr=True)


def gaussian_blur(img: Image, kx: int, ky=None, sigma: float = None) -> Image:
    """``gaussian_blur(img, ksize, sigma)`` or ``gaussian_blur(img, kx, ky, sigma)``."""
    if sigma is None:
        kx, ky, sigma = kx, kx, (0.0 if ky is None else ky)
    kx, ky = _odd(kx), _odd(ky)
    return _like(img, K.gaussian_blur(img.ensure_packed_hwc_u8().data, kx, ky, max(float(sigma), 0.0)))


def median_blur(img: Image, ksize: int) -> Image:
    k = _odd(ksize)
    if img.data.is_cuda and k <= 9:
        return _like(img, K.median(img.ensure_packed_hwc_u8().data, k))
    r = k // 2
    a = img.numpy()
    p = np.pad(a, ((r, r), (r, r), (0, 0)), mode="edge")
    h, w = a.shape[:2]
    stack = np.stack([p[dy:dy + h, dx:dx + w] for dy in range(k) for dx in range(k)], 0)
    return _like(img, torch.from_numpy(np.median(stack, axis=0).astype(np.uint8)).to(img.device))


def bilateral_filter(img: Image, d: int, sigma_color: float, sigma_space: float) -> Image:
    d = _odd(d if d > 0 else int(round(sigma_space * 1.5)) * 2 + 1, 3)
    r = d // 2
    if img.data.is_cuda and img.ensure_packed_hwc_u8().data.shape[2] <= 4:
        return _like(img, K.bilateral(img.ensure_packed_hwc_u8().data, r, sigma_color, sigma_space))
    a = img.numpy().astype(np.float32)
    h, w = a.shape[:2]
    p = np.pad(a, ((r, r), (r, r), (0, 0)), mode="edge")
    num = np.zeros_like(a)
    den = np.zeros(a.shape[:2] + (1,), dtype=np.float32)
    sc2 = 2.0 * max(float(sigma_color), 1e-6) ** 2
    ss2 = 2.0 * max(float(sigma_space), 1e-6) ** 2
    for dy in range(-r, r + 1):
        for dx in range(-r, r + 1):
            q = p[r + dy:r + dy + h, r + dx:r + dx + w]
            diff = np.abs(q - a).sum(-1, keepdims=True)
            wgt = np.exp(-(diff * diff) / sc2 - (dx * dx + dy * dy) / ss2).astype(np.float32)
            num += wgt * q
            den += wgt
    out = np.clip(num / den + 0.5, 0, 255).astype(np.uint8)
    return _like(img, torch.from_numpy(out).to(img.device))


bilateral_blur = bilateral_filter


def sobel(img: Image, dx: int, dy: int, ksize: int = 3) -> Image:
    """|d/dx| if dx > 0 (and dy == 0), |d/dy| if dy > 0, gradient magnitude if both; 3x3 kernels."""
    g = _gray_data(img)
    mode = K.DERIV_MAGNITUDE if (dx > 0 and dy > 0) else (K.DERIV_SOBEL_Y if dy > 0 else K.DERIV_SOBEL_X)
    return _like(img, K.deriv3(g, mode))


def laplacian(img: Image, ksize: int = 3) -> Image:
    return _like(img, K.deriv3(_gray_data(img), K.DERIV_LAPLACE))


def magnitude_u8(gx: Image, gy: Image) -> Image:
    h, w = min(gx.height(), gy.height()), min(gx.width(), gy.width())
    if h <= 0 or w <= 0:
        return Image.new_hwc_u8(1, 1, 1, 0)
    a = gx.data[:h, :w, 0].to(torch.float32)
    b = gy.data[:h, :w, 0].to(torch.float32)
    return Image(torch.sqrt(a * a + b * b).clamp(0, 255).to(torch.uint8).unsqueeze(-1))


def canny(img: Image, t1: int, t2: int, aperture: int = 3) -> Image:
    lo, hi = (t1, t2) if t1 <= t2 else (t2, t1)
    if img.data.is_cuda:
        return Image(K.canny(_gray_data(img), lo, hi))
    g = _gray_data(img).cpu().numpy()[..., 0].astype(np.int32)
    h, w = g.shape
    p = np.pad(g, 1, mode="edge")
    s = lambda dy, dx: p[1 + dy:1 + dy + h, 1 + dx:1 + dx + w]
    gx = (s(-1, 1) + 2 * s(0, 1) + s(1, 1)) - (s(-1, -1) + 2 * s(0, -1) + s(1, -1))
    gy = (s(1, -1) + 2 * s(1, 0) + s(1, 1)) - (s(-1, -1) + 2 * s(-1, 0) + s(-1, 1))
    mag = np.abs(gx) + np.abs(gy)
    ang = (np.rad2deg(np.arctan2(gy, gx)) + 180.0) % 180.0
    sector = ((ang + 22.5) // 45).astype(np.int64) % 4
    mp = np.pad(mag, 1, mode="constant")
    m = lambda dy, dx: mp[1 + dy:1 + dy + h, 1 + dx:1 + dx + w]
    n1 = np.choose(sector, [m(0, 1), m(1, 1), m(1, 0), m(1, -1)])
    n2 = np.choose(sector, [m(0, -1), m(-1, -1), m(-1, 0), m(-1, 1)])
    nms = np.where((mag >= n1) & (mag >= n2), mag, 0)
    strong = nms >= hi
    weak = (nms >= lo) & ~strong
    out = strong.copy()
    stack = list(zip(*np.nonzero(strong)))
    while stack:
        y, x = stack.pop()
        for dy in (-1, 0, 1):
            for dx in (-1, 0, 1):
                yy, xx = y + dy, x + dx
                if 0 <= yy < h and 0 <= xx < w and weak[yy, xx] and not out[yy, xx]:
                    out[yy, xx] = True
                    stack.append((yy, xx))
    return Image(torch.from_numpy((out * 255).astype(np.uint8)[..., None]).to(img.device))


def ones_u8(h: int, w: int) -> Image:
    if h <= 0 or w <= 0:
        return Image.new_hwc_u8(1, 1, 1, 1)
    return Image.new_hwc_u8(h, w, 1, 1)
