"""Colour conversions and histogram tools (legacy/src/momijo/vision/transforms/color.mojo)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from ..image import ColorSpace, Image
from .. import kernels as K


def _like(img, data, cs=None):
    meta = img.meta().copy()
    if cs is not None:
        meta = meta.with_colorspace(cs)
    return Image(data, meta)


def bgr_to_rgb(img: Image) -> Image:
    return _like(img, K.swap_rb(img.ensure_packed_hwc_u8().data), ColorSpace("RGB"))


def rgb_to_bgr(img: Image) -> Image:
    return _like(img, K.swap_rb(img.ensure_packed_hwc_u8().data), ColorSpace("BGR"))


def bgr_to_gray(img: Image) -> Image:
    return _like(img, K.to_gray(img.ensure_packed_hwc_u8().data, bgr=True), ColorSpace("GRAY"))


def rgb_to_gray(img: Image) -> Image:
    """gray = (299 R + 587 G + 114 B) / 1000 in integers
    (legacy/src/momijo/vision/backend/cpu/convert_color_cpu.mojo:45)."""
    return _like(img, K.to_gray(img.ensure_packed_hwc_u8().data, bgr=False), ColorSpace("GRAY"))


def gray_to_bgr(img: Image) -> Image:
    return _like(img, img.data[..., :1].expand(-1, -1, 3).contiguous(), ColorSpace("BGR"))


def split3(img: Image) -> Tuple[Image, Image, Image]:
    d = img.data
    return tuple(Image(d[..., k:k + 1].contiguous()) for k in range(3))


def merge3(r: Image, g: Image, b: Image) -> Image:
    return Image(torch.cat([r.data[..., :1], g.data[..., :1], b.data[..., :1]], -1).contiguous())


def histogram(img, bins: int = 256) -> List[int]:
    """Counts of channel 0 in ``bins`` equal-width bins over 0..255."""
    if isinstance(img, Image):
        h = K.histogram(img.ensure_packed_hwc_u8().data, 0).cpu().numpy()
    else:
        h = np.bincount(np.asarray(img, dtype=np.uint8).reshape(-1), minlength=256)
    bins = max(1, min(int(bins), 256))
    if bins == 256:
        return [int(v) for v in h]
    out = [0] * bins
    for v in range(256):
        out[(v * bins) // 256] += int(h[v])
    return out


def _equalize_lut(hist: np.ndarray) -> np.ndarray:
    cdf = np.cumsum(hist.astype(np.int64))
    total = int(cdf[-1])
    nz = np.nonzero(cdf)[0]
    cdf_min = int(cdf[nz[0]]) if len(nz) else 0
    denom = total - cdf_min
    if denom <= 0:
        return np.arange(256, dtype=np.uint8)
    return np.clip(((cdf - cdf_min) * 255) // denom, 0, 255).astype(np.uint8)


def equalize_hist(img: Image) -> Image:
    x = img.ensure_packed_hwc_u8()
    if x.channels() != 1 or x.is_empty():
        return x.clone()
    hist = K.histogram(x.data, 0).cpu().numpy()
    return _like(img, K.apply_lut(x.data, _equalize_lut(hist)))


def plot_hist_u8(hist: Sequence[int], width: int = 256, height: int = 200) -> Image:
    out = np.zeros((height, width, 1), dtype=np.uint8)
    n = len(hist)
    peak = max(max(hist), 1) if n else 1
    for x in range(width):
        v = hist[min((x * n) // width, n - 1)] if n else 0
        bar = (int(v) * (height - 1)) // peak
        if bar > 0:
            out[height - bar:, x, 0] = 255
    return Image(torch.from_numpy(out))


def _clahe_plane(a: np.ndarray, clip_limit: float, tile: int) -> np.ndarray:
    h, w = a.shape
    ty, tx = max(1, min(tile, h)), max(1, min(tile, w))
    ys = np.linspace(0, h, ty + 1).astype(int)
    xs = np.linspace(0, w, tx + 1).astype(int)
    luts = np.zeros((ty, tx, 256), dtype=np.float32)
    for i in range(ty):
        for j in range(tx):
            blk = a[ys[i]:ys[i + 1], xs[j]:xs[j + 1]]
            hist = np.bincount(blk.reshape(-1), minlength=256).astype(np.float64)
            limit = max(1.0, clip_limit * blk.size / 256.0)
            excess = np.maximum(hist - limit, 0).sum()
            hist = np.minimum(hist, limit) + excess / 256.0
            cdf = np.cumsum(hist)
            luts[i, j] = cdf * 255.0 / max(cdf[-1], 1.0)
    cy = (ys[:-1] + ys[1:]) / 2.0
    cx = (xs[:-1] + xs[1:]) / 2.0
    yy = np.arange(h)[:, None] + 0.5
    xx = np.arange(w)[None, :] + 0.5
    fi = np.clip(np.interp(yy[:, 0], cy, np.arange(ty)), 0, ty - 1)
    fj = np.clip(np.interp(xx[0], cx, np.arange(tx)), 0, tx - 1)
    i0, j0 = np.floor(fi).astype(int), np.floor(fj).astype(int)
    i1, j1 = np.minimum(i0 + 1, ty - 1), np.minimum(j0 + 1, tx - 1)
    wy, wx = (fi - i0)[:, None], (fj - j0)[None, :]
    g = lambda ii, jj: luts[ii[:, None], jj[None, :], a]
    v = (g(i0, j0) * (1 - wx) + g(i0, j1) * wx) * (1 - wy) + (g(i1, j0) * (1 - wx) + g(i1, j1) * wx) * wy
    return np.clip(v + 0.5, 0, 255).astype(np.uint8)


def clahe_color_bgr(img, clip_limit: float = 2.0, tile: int = 8):
    """Contrast-limited adaptive equalisation of the luma of a BGR image; chroma is kept."""
    is_img = isinstance(img, Image)
    if is_img and img.data.is_cuda:
        d = img.ensure_packed_hwc_u8().data
        if d.shape[2] == 1:
            out_t = K.clahe_plane(d[..., 0], clip_limit, tile).unsqueeze(-1)
        else:
            f = d[..., :3].to(torch.float32)
            y = f[..., 2] * 0.299 + f[..., 1] * 0.587 + f[..., 0] * 0.114
            y8 = (y + 0.5).clamp(0, 255).to(torch.uint8)
            y2 = K.clahe_plane(y8, clip_limit, tile).to(torch.float32)
            out_t = (f + (y2 - y).unsqueeze(-1) + 0.5).clamp(0, 255).to(torch.uint8)
            if d.shape[2] > 3:
                out_t = torch.cat([out_t, d[..., 3:]], dim=-1)
        return Image(out_t.contiguous(), img.meta().copy())
    a = img.numpy() if is_img else np.asarray(img, dtype=np.uint8)
    if a.ndim == 2 or a.shape[2] == 1:
        out = _clahe_plane(a.reshape(a.shape[0], a.shape[1]), clip_limit, tile)[..., None]
    else:
        f = a[..., :3].astype(np.float32)
        y = (f[..., 2] * 0.299 + f[..., 1] * 0.587 + f[..., 0] * 0.114)
        y8 = np.clip(y + 0.5, 0, 255).astype(np.uint8)
        y2 = _clahe_plane(y8, clip_limit, tile).astype(np.float32)
        out = np.clip(f + (y2 - y)[..., None] + 0.5, 0, 255).astype(np.uint8)
    if is_img:
        return Image(torch.from_numpy(np.ascontiguousarray(out)).to(img.device), img.meta().copy())
    return out.tolist()


def color_jitter(img: Image, brightness: float, contrast: float, saturation: float, hue: float) -> Image:
    """``ColorJitter(brightness, contrast, saturation, hue)(img)``: multiplicative brightness and contrast
    factors (1.0 = unchanged), saturation factor, hue shift in degrees
    (legacy/src/momijo/vision/transforms/color.mojo:622-625)."""
    from .random_ops import ColorJitter
    return ColorJitter(brightness, contrast, saturation, hue)(img)
