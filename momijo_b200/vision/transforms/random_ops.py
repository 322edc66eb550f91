"""Stateful augmentation transforms and small tensor adapters of the vision package.

``ColorJitter`` (legacy/src/momijo/vision/transforms/color.mojo:454-625), ``RandomHorizontalFlip`` and
``RandomRotation`` (legacy/src/momijo/vision/transforms/geom.mojo:102-275), ``RandomResizedCrop`` and
``resize_nearest_u8_hwc`` (legacy/src/momijo/vision/transforms/resize.mojo:20-165), ``ToTensor``
(legacy/src/momijo/vision/tensor.mojo:408-424), ``Keypoint`` (legacy/src/momijo/vision/transforms/features.mojo:10-34).

Every transform takes an ``Image`` (or a packed HWC uint8 torch tensor) and returns the same kind of
object; the pixel arithmetic runs as torch ops on the tensor's device, so CUDA images stay on the GPU.
The random ones keep the reference's 64-bit LCG (state * 6364136223846793005 + 1, bits 33..64 as a
uniform in [0, 1)), so a given seed yields the same decisions as the reference."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..image import Image

_MASK64 = (1 << 64) - 1


class _LCG:
    def __init__(self, seed: int):
        self._state = int(seed) & _MASK64

    def rand01(self) -> float:
        self._state = (self._state * 6364136223846793005 + 1) & _MASK64
        return ((self._state >> 33) & 0xFFFFFFFF) / 4294967296.0

    def uniform(self, a: float, b: float) -> float:
        return a + (b - a) * self.rand01()

    def randint(self, lo: int, hi_exclusive: int) -> int:
        span = hi_exclusive - lo
        assert span > 0, "randint: invalid range"
        return lo + min(int(self.rand01() * span), span - 1)


def _data(x) -> torch.Tensor:
    return x.ensure_packed_hwc_u8().data if isinstance(x, Image) else x


def _back(x, data: torch.Tensor):
    return Image(data.contiguous(), x.meta().copy()) if isinstance(x, Image) else data.contiguous()


# ---- colour jitter ---------------------------------------------------------------------------------
def _rgb_to_hsv(r, g, b):
    rf, gf, bf = r / 255.0, g / 255.0, b / 255.0
    maxv = torch.maximum(rf, torch.maximum(gf, bf))
    minv = torch.minimum(rf, torch.minimum(gf, bf))
    d = maxv - minv
    s = torch.where(maxv > 0, d / maxv.clamp_min(1e-30), torch.zeros_like(d))
    dd = torch.where(d != 0, d, torch.ones_like(d))
    h = torch.where(maxv == rf, 60.0 * torch.remainder((gf - bf) / dd, 6.0),
                    torch.where(maxv == gf, 60.0 * ((bf - rf) / dd + 2.0), 60.0 * ((rf - gf) / dd + 4.0)))
    h = torch.where(d != 0, h, torch.zeros_like(h))
    h = torch.where(h < 0, h + 360.0, h)
    return h, s, maxv


def _hsv_to_rgb(h, s, v):
    hh = h / 60.0
    i = hh.floor()
    f = hh - i
    p, q, t = v * (1.0 - s), v * (1.0 - s * f), v * (1.0 - s * (1.0 - f))
    i = i.long().clamp(0, 5)
    r = torch.stack([v, q, p, p, t, v], 0).gather(0, i[None])[0]
    g = torch.stack([t, v, v, q, p, p], 0).gather(0, i[None])[0]
    b = torch.stack([p, p, t, v, v, q], 0).gather(0, i[None])[0]
    grey = s == 0
    return (torch.where(grey, v, r) * 255.0, torch.where(grey, v, g) * 255.0, torch.where(grey, v, b) * 255.0)


class ColorJitter:
    """Deterministic colour adjustment: brightness and contrast are multiplicative factors (1.0 leaves the
    image alone; contrast pivots on 128), saturation scales S in HSV and ``hue`` is a shift in degrees.
    Grey images get brightness and contrast only; channels beyond the third are copied through."""

    def __init__(self, brightness: float, contrast: float, saturation: float, hue: float):
        self._brightness, self._contrast = float(brightness), float(contrast)
        self._saturation, self._hue_deg = float(saturation), float(hue)

    def __call__(self, x):
        src = _data(x)
        assert src.dtype == torch.uint8 and src.dim() == 3, "ColorJitter: packed HWC uint8 input"
        f = src.float()
        c = f.shape[2]
        if c < 3:
            v = (f * self._brightness - 128.0) * self._contrast + 128.0
            return _back(x, (v.clamp(0, 255) + 0.5).to(torch.uint8))
        rgb = f[..., :3]
        if self._brightness != 1.0:
            rgb = rgb * self._brightness
        if self._contrast != 1.0:
            rgb = (rgb - 128.0) * self._contrast + 128.0
        r, g, b = rgb[..., 0], rgb[..., 1], rgb[..., 2]
        if self._saturation != 1.0 or self._hue_deg != 0.0:
            h, s, v = _rgb_to_hsv(r, g, b)
            s = (s * self._saturation).clamp(0.0, 1.0)
            h = torch.remainder(h + self._hue_deg, 360.0)
            r, g, b = _hsv_to_rgb(h, s, v)
        out = src.clone()
        out[..., :3] = (torch.stack([r, g, b], -1).clamp(0, 255) + 0.5).to(torch.uint8)
        return _back(x, out)


# ---- geometry ----------------------------------------------------------------------------------------
class RandomHorizontalFlip:
    """Mirrors the image left-right with probability ``p``; one generator draw per call. Images and uint8
    tensors are HWC (the width is axis 1); float tensors are taken as CHW like the reference's float path
    (the width is the last axis)."""

    def __init__(self, p: float = 0.5, seed: int = 88172645463325252):
        self.p = p
        self._rng = _LCG(seed)

    def __call__(self, x):
        src = _data(x)
        flip = self._rng.rand01() < self.p
        w_axis = -1 if (src.is_floating_point() or src.dim() != 3) else 1
        return _back(x, torch.flip(src, [w_axis]) if flip else src.clone())


def _rotate_nearest_hwc_u8(src: torch.Tensor, angle_deg: float) -> torch.Tensor:
    """Rotation about the image centre, nearest neighbour, zero outside (inverse mapping, the same
    rounding as the reference)."""
    h, w = src.shape[0], src.shape[1]
    cx, cy = (w - 1) * 0.5, (h - 1) * 0.5
    t = math.radians(angle_deg)
    ct, st = math.cos(t), math.sin(t)
    oy, ox = torch.meshgrid(torch.arange(h, device=src.device, dtype=torch.float64),
                            torch.arange(w, device=src.device, dtype=torch.float64), indexing="ij")
    dx, dy = ox - cx, oy - cy
    # round half away from zero, like round() on the reference side
    rnd = lambda v: torch.where(v >= 0, (v + 0.5).floor(), (v - 0.5).ceil())
    sx = rnd(dx * ct + dy * st + cx).long()
    sy = rnd(-dx * st + dy * ct + cy).long()
    inside = (sx >= 0) & (sx < w) & (sy >= 0) & (sy < h)
    out = src[sy.clamp(0, h - 1), sx.clamp(0, w - 1)]
    return torch.where(inside[..., None], out, torch.zeros_like(out))


class RandomRotation:
    """With probability ``p`` rotates by an angle drawn uniformly from [-degrees, +degrees]."""

    def __init__(self, degrees: float, p: float = 1.0, seed: int = 0xC0FFEE1234):
        assert degrees >= 0.0, "RandomRotation: degrees must be non-negative"
        self.degrees, self.p = float(degrees), p
        self._rng = _LCG(seed)

    def __call__(self, x):
        src = _data(x)
        if self._rng.rand01() >= self.p:
            return _back(x, src.clone())
        angle = self._rng.uniform(-self.degrees, self.degrees)
        return _back(x, _rotate_nearest_hwc_u8(src, angle))


def resize_nearest_u8_hwc(x, out_h: int, out_w: int):
    """Nearest-neighbour resize with source index int(y * h / out_h), clamped."""
    src = _data(x)
    h, w = src.shape[0], src.shape[1]
    assert out_h > 0 and out_w > 0, "resize_nearest_u8_hwc: bad output shape"
    ys = (torch.arange(out_h, device=src.device, dtype=torch.float64) * (h / out_h)).long().clamp(0, h - 1)
    xs = (torch.arange(out_w, device=src.device, dtype=torch.float64) * (w / out_w)).long().clamp(0, w - 1)
    out = src[ys][:, xs]
    if isinstance(x, Image):
        return Image(out.contiguous(), x.meta().copy())
    return out.contiguous()


class RandomResizedCrop:
    """Random ``out_h x out_w`` window when the image is at least that large, else a nearest-neighbour resize
    to the target size (no randomness)."""

    def __init__(self, out_h: int, out_w: int, seed: int = 0x9E3779B97F4A7C15):
        self.out_h, self.out_w = out_h, out_w
        self._rng = _LCG(seed)

    def __call__(self, x):
        src = _data(x)
        h, w = src.shape[0], src.shape[1]
        if h >= self.out_h and w >= self.out_w:
            top = self._rng.randint(0, h - self.out_h + 1)
            left = self._rng.randint(0, w - self.out_w + 1)
            out = src[top:top + self.out_h, left:left + self.out_w].clone()
            return Image(out, x.meta().copy()) if isinstance(x, Image) else out
        return resize_nearest_u8_hwc(x, self.out_h, self.out_w)


def random_resized_crop(x, out_h: int, out_w: int, seed: int = 0x9E3779B97F4A7C15):
    return RandomResizedCrop(out_h, out_w, seed)(x)


# ---- adapters ----------------------------------------------------------------------------------------
class ToTensor:
    """HWC uint8 -> float32 scaled by ``scale`` (default 1/255), CHW by default or HWC with
    ``to_chw=False``. Invalid shapes give an empty tensor."""

    def __init__(self, scale: float = 1.0 / 255.0, to_chw: bool = True):
        self._scale, self._to_chw = float(scale), bool(to_chw)

    def __call__(self, x, h: int = None, w: int = None, c: int = None):
        src = _data(x)
        if h is not None:
            if h <= 0 or w <= 0 or c <= 0:
                return torch.zeros(0)
            src = src.reshape(h, w, c)
        if src.dim() == 2:
            src = src[..., None]
        if src.numel() == 0:
            return torch.zeros(0)
        out = src.float() * self._scale
        return out.permute(2, 0, 1).contiguous() if self._to_chw else out


@dataclass
class Keypoint:
    x: int
    y: int
    size: float = 0.0
    angle: float = -1.0
    response: float = 0.0
    octave: int = 0
    class_id: int = -1


def random_affine_placeholder(x, degrees: float, tx: float, ty: float, smin: float, smax: float):
    """Identity: the reference's hook for a future affine augmentation
    (legacy/src/momijo/vision/transforms/transforms.mojo:56-63); ``Compose.add_random_affine`` is the real one."""
    return x


def maybe_resize_placeholder(x, img_size: int):
    """Identity copy (legacy/src/momijo/vision/transforms/transforms.mojo:66-69)."""
    return x.clone() if hasattr(x, "clone") else x


def abs_f64(v: float) -> float:
    return -v if v < 0 else v


def resize_nearest_u8_hwc_tiled_scheduled(x, out_h: int, out_w: int, sched=None):
    """Same pixels as ``resize_nearest_u8_hwc``; the schedule only sets the tile walk of the host loop in the
    reference (legacy/src/momijo/vision/transforms/tile.mojo:24-90) and the launch shape of the CUDA kernel
    here, so it cannot change the result."""
    return resize_nearest_u8_hwc(x, out_h, out_w)


def resize_nearest_u8_hwc_tiled(x, out_h: int, out_w: int):
    return resize_nearest_u8_hwc(x, out_h, out_w)
