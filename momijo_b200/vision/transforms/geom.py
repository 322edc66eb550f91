"""Geometric transforms (legacy/src/momijo/vision/transforms/geom.mojo). The reference's
``resize``/``rotate`` only allocate blank outputs of the right shape (geom.mojo:32-61); here they
resample. Warps sample the nearest source pixel at floor(M^-1 [x y 1] + 0.5), the reference's
``_warp_affine``/``_warp_perspective`` scheme (geom.mojo:586-640) with the rounding made symmetric."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..image import Image
from .. import kernels as K


@dataclass
class BorderSpec:
    mode: int = 0
    value: int = 0

    def cval(self) -> int:
        return self.value

    @staticmethod
    def CONSTANT(val: int = 0):
        return BorderSpec(0, int(val))

    @staticmethod
    def REPLICATE():
        return BorderSpec(1, 0)

    @staticmethod
    def REFLECT():
        return BorderSpec(2, 0)


def BORDER_CONSTANT_BS(val=0): return BorderSpec.CONSTANT(val)
def BORDER_REPLICATE_BS(): return BorderSpec.REPLICATE()
def BORDER_REFLECT_BS(): return BorderSpec.REFLECT()
def BORDER_CONSTANT(): return 0
def BORDER_REPLICATE(): return 1
def BORDER_REFLECT(): return 2
def INTER_NEAREST(): return 2
def INTER_LINEAR(): return 0
def INTER_AREA(): return 1
def MORPH_OPEN(): return 0
def MORPH_CLOSE(): return 1
def MORPH_GRADIENT(): return 2
def ADAPTIVE_GAUSSIAN(): return 0
def FONT_PLAIN(): return 0
def FONT_SIMPLEX(): return 1


def to_border_spec(code, val: int = 0) -> BorderSpec:
    if isinstance(code, BorderSpec):
        return code
    return BorderSpec(int(code) if int(code) in (0, 1, 2) else 0, int(val))


def deg2rad(deg: float) -> float:
    return float(deg) * math.pi / 180.0


def _like(img: Image, data: torch.Tensor) -> Image:
    return Image(data, img.meta().copy())


def resize(img: Image, new_w: int, new_h: int, inter: int = 0) -> Image:
    """``inter``: INTER_LINEAR (0, default) and INTER_AREA (1) interpolate bilinearly, 2 is nearest."""
    W = new_w if new_w > 0 else img.width()
    H = new_h if new_h > 0 else img.height()
    return _like(img, K.resize(img.ensure_packed_hwc_u8().data, H, W, bilinear=(inter != 2)))


def resize_nearest(img: Image, out_h: int, out_w: int) -> Image:
    return _like(img, K.resize(img.ensure_packed_hwc_u8().data, out_h, out_w, bilinear=False))


def crop(img: Image, y: int, x: int, h: int, w: int) -> Image:
    return Image(img.roi(y, x, h, w).data.clone(), img.meta().copy())


def flip(img: Image, axis: int = 0) -> Image:
    """axis 0: vertical (rows reversed), 1: horizontal, -1: both."""
    dims = [0] if axis == 0 else ([1] if axis == 1 else [0, 1])
    return _like(img, torch.flip(img.data, dims).contiguous())


def rotate90(img: Image, k=1) -> Image:
    """``k`` counts counter-clockwise quarter turns; a bool means clockwise or not."""
    if isinstance(k, bool):
        k = -1 if k else 1
    return _like(img, torch.rot90(img.data, int(k) % 4, (0, 1)).contiguous())


def _inv3(m):
    a = np.asarray(m, dtype=np.float64).reshape(3, 3)
    if np.linalg.det(a) == 0.0:
        return None
    return np.linalg.inv(a).reshape(-1).tolist()


def _warp(img: Image, M: Sequence[float], perspective_: bool, border) -> Image:
    inv = _inv3(M)
    if inv is None:
        return img.clone()
    bs = to_border_spec(border)
    return _like(img, K.warp(img.ensure_packed_hwc_u8().data, inv, perspective_, bs.mode, bs.value))


def translate(img: Image, dx: int, dy: int, border=0) -> Image:
    return _warp(img, [1, 0, dx, 0, 1, dy, 0, 0, 1], False, border)


def rotate(img: Image, angle: float, scale: float = 1.0, center_x: float = -1.0, center_y: float = -1.0,
           border=0) -> Image:
    """Counter-clockwise rotation by ``angle`` degrees about the centre (default: image centre)."""
    a = float(angle) % 360.0
    if scale == 1.0 and center_x < 0 and center_y < 0 and a in (0.0, 90.0, 180.0, 270.0):
        return rotate90(img, int(a // 90))
    cx = (img.width() - 1) / 2.0 if center_x < 0 else center_x
    cy = (img.height() - 1) / 2.0 if center_y < 0 else center_y
    t = deg2rad(angle)
    al, be = scale * math.cos(t), scale * math.sin(t)
    M = [al, be, (1 - al) * cx - be * cy, -be, al, be * cx + (1 - al) * cy, 0, 0, 1]
    return _warp(img, M, False, border)


rotate_basic = rotate


def _affine_from_3pts(src, dst):
    A = np.array([[x, y, 1.0] for x, y in src], dtype=np.float64)
    if np.linalg.det(A) == 0.0:
        return None
    X = np.array([p[0] for p in dst], dtype=np.float64)
    Y = np.array([p[1] for p in dst], dtype=np.float64)
    Ai = np.linalg.inv(A)
    return list(Ai @ X) + list(Ai @ Y) + [0.0, 0.0, 1.0]


def _solve_homography(src, dst):
    rows, b = [], []
    for (x, y), (X, Y) in zip(src, dst):
        rows.append([x, y, 1, 0, 0, 0, -x * X, -y * X]); b.append(X)
        rows.append([0, 0, 0, x, y, 1, -x * Y, -y * Y]); b.append(Y)
    A = np.array(rows, dtype=np.float64)
    if abs(np.linalg.det(A)) < 1e-12:
        return None
    return list(np.linalg.solve(A, np.array(b, dtype=np.float64))) + [1.0]


def _pts(p):
    p = list(p)
    if p and not isinstance(p[0], (tuple, list)):
        p = [(p[i], p[i + 1]) for i in range(0, len(p), 2)]
    return [(float(a), float(b)) for a, b in p]


def affine(img: Image, a, b=None, border=0) -> Image:
    """Either ``affine(img, M)`` with a 2x3 / 3x3 matrix (flat or nested) or ``affine(img, src3, dst3)``
    with three point pairs."""
    if b is None or isinstance(b, (int, BorderSpec)):
        if isinstance(b, (int, BorderSpec)):
            border = b
        m = np.asarray(a, dtype=np.float64).reshape(-1).tolist()
        M = m + [0.0, 0.0, 1.0] if len(m) == 6 else m
    else:
        M = _affine_from_3pts(_pts(a), _pts(b))
        if M is None:
            return img.clone()
    return _warp(img, M, False, border)


def perspective(img: Image, a, b=None, border=0) -> Image:
    """``perspective(img, H)`` with a 3x3 matrix or ``perspective(img, src4, dst4)``."""
    if b is None or isinstance(b, (int, BorderSpec)):
        if isinstance(b, (int, BorderSpec)):
            border = b
        M = np.asarray(a, dtype=np.float64).reshape(-1).tolist()
    else:
        M = _solve_homography(_pts(a), _pts(b))
        if M is None:
            return img.clone()
    return _warp(img, M, True, border)


def copy_make_border(img: Image, top: int, bottom: int, left: int, right: int, border=0, value: int = 0) -> Image:
    bs = to_border_spec(border, value)
    a = img.numpy()
    pad = ((max(top, 0), max(bottom, 0)), (max(left, 0), max(right, 0)), (0, 0))
    if bs.mode == 1:
        out = np.pad(a, pad, mode="edge")
    elif bs.mode == 2:
        out = np.pad(a, pad, mode="reflect") if min(a.shape[:2]) > 1 else np.pad(a, pad, mode="edge")
    else:
        out = np.pad(a, pad, mode="constant", constant_values=bs.value)
    return Image(torch.from_numpy(np.ascontiguousarray(out)).to(img.device), img.meta().copy())


def random_horizontal_flip(img, p=0.5, seed=0xC0FFEE1234, w: int = None, p_ref: float = 0.5, seed_ref: int = 88172645463325252):
    """``random_horizontal_flip(image, p, seed)``. The reference's raw-buffer form ``(data, c, h, w, p, seed)``
    (legacy/src/momijo/vision/transforms/geom.mojo:144-147) takes a float [C, H, W] tensor (or flat buffer) and goes
    through ``RandomHorizontalFlip``."""
    if w is not None:
        from .random_ops import RandomHorizontalFlip
        import torch
        buf = torch.as_tensor(img, dtype=torch.float32).reshape(int(p), int(seed), int(w))
        return RandomHorizontalFlip(p_ref, seed_ref)(buf)
    state = (int(seed) * 6364136223846793005 + 1) & ((1 << 64) - 1)
    r = ((state >> 33) & 0xFFFFFFFF) / 4294967296.0
    return flip(img, 1) if r < p else img.clone()


def random_rotation(img: Image, degrees: float, p: float = 1.0, seed: int = 0xC0FFEE1234) -> Image:
    state = (int(seed) * 6364136223846793005 + 1) & ((1 << 64) - 1)
    r1 = ((state >> 33) & 0xFFFFFFFF) / 4294967296.0
    state = (state * 6364136223846793005 + 1) & ((1 << 64) - 1)
    r2 = ((state >> 33) & 0xFFFFFFFF) / 4294967296.0
    if r1 >= p:
        return img.clone()
    return rotate(img, (2.0 * r2 - 1.0) * degrees)
