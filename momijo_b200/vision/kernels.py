"""Pixel kernels behind the transforms: each function takes and returns packed HWC uint8 torch
tensors. Tensors in device memory run the CUDA kernels of ``csrc/vision.cu``; tensors in host memory
run a vectorised restatement of the same arithmetic (the oracle the GPU tests compare against).

Reference loops restated here: nearest resize (legacy/src/momijo/vision/backend/cpu/
resize_cpu.mojo:22-55), grey conversion (legacy/src/momijo/vision/backend/cpu/
convert_color_cpu.mojo:20-48), separable gaussian (legacy/src/momijo/vision/transforms/
filter.mojo:62-171), erode/dilate (legacy/src/momijo/vision/transforms/morph.mojo:66-140),
warps (legacy/src/momijo/vision/transforms/geom.mojo:586-640).
"""
from __future__ import annotations

import ctypes
import math
from typing import Sequence

import numpy as np
import torch

from .. import _C

BORDER_CONSTANT, BORDER_REPLICATE, BORDER_REFLECT = 0, 1, 2


def _prep(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.uint8:
        raise TypeError("vision kernels work on uint8 images")
    if t.dim() == 2:
        t = t.unsqueeze(-1)
    return t.contiguous()


def _launch(name, *args):
    rc = _C.call(name, *args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


def _stream():
    return _C.current_stream()


# ---- resize --------------------------------------------------------------------------------------
def resize(src: torch.Tensor, oh: int, ow: int, bilinear: bool = False) -> torch.Tensor:
    src = _prep(src)
    ih, iw, c = src.shape
    if src.is_cuda:
        dst = torch.empty((oh, ow, c), dtype=torch.uint8, device=src.device)
        _launch("mmj_vis_resize", _C.ptr(src), _C.ptr(dst), ih, iw, c, oh, ow, int(bilinear), _stream())
        return dst
    a = src.numpy()
    if not bilinear:
        ys = np.clip((np.arange(oh) * (ih / oh)).astype(np.int64), 0, ih - 1)
        xs = np.clip((np.arange(ow) * (iw / ow)).astype(np.int64), 0, iw - 1)
        return torch.from_numpy(np.ascontiguousarray(a[ys][:, xs]))
    sy, sx = np.float32(ih) / np.float32(oh), np.float32(iw) / np.float32(ow)
    fy = np.clip((np.arange(oh, dtype=np.float32) + np.float32(0.5)) * sy - np.float32(0.5), 0, ih - 1).astype(np.float32)
    fx = np.clip((np.arange(ow, dtype=np.float32) + np.float32(0.5)) * sx - np.float32(0.5), 0, iw - 1).astype(np.float32)
    y0, x0 = fy.astype(np.int64), fx.astype(np.int64)
    y1, x1 = np.minimum(y0 + 1, ih - 1), np.minimum(x0 + 1, iw - 1)
    wy = (fy - y0).astype(np.float32)[:, None, None]
    wx = (fx - x0).astype(np.float32)[None, :, None]
    f = a.astype(np.float32)
    one = np.float32(1.0)
    top = f[y0][:, x0] * (one - wx) + f[y0][:, x1] * wx
    bot = f[y1][:, x0] * (one - wx) + f[y1][:, x1] * wx
    v = top * (one - wy) + bot * wy
    return torch.from_numpy((v + np.float32(0.5)).astype(np.uint8))


# ---- colour --------------------------------------------------------------------------------------
def to_gray(src: torch.Tensor, bgr: bool = False) -> torch.Tensor:
    src = _prep(src)
    h, w, c = src.shape
    if c < 3:
        return src[..., :1].clone()
    if src.is_cuda:
        dst = torch.empty((h, w, 1), dtype=torch.uint8, device=src.device)
        _launch("mmj_vis_to_gray", _C.ptr(src), _C.ptr(dst), h * w, c, int(bgr), _stream())
        return dst
    a = src.numpy().astype(np.int32)
    r, g, b = (a[..., 2], a[..., 1], a[..., 0]) if bgr else (a[..., 0], a[..., 1], a[..., 2])
    return torch.from_numpy(((r * 299 + g * 587 + b * 114) // 1000).astype(np.uint8)[..., None])


def swap_rb(src: torch.Tensor) -> torch.Tensor:
    src = _prep(src)
    h, w, c = src.shape
    if c < 3:
        return src.clone()
    if src.is_cuda:
        dst = torch.empty_like(src)
        _launch("mmj_vis_swap_rb", _C.ptr(src), _C.ptr(dst), h * w, c, _stream())
        return dst
    idx = [2, 1, 0] + list(range(3, c))
    return src[..., idx].contiguous()


# ---- separable gaussian ----------------------------------------------------------------------------
def gaussian_taps(ksize: int, sigma: float) -> np.ndarray:
    r = ksize // 2
    d = np.arange(-r, r + 1, dtype=np.float64)
    w = np.exp(-(d * d) / (2.0 * sigma * sigma)) if sigma > 0 else np.ones_like(d)
    return (w / w.sum())


def sigma_from_ksize(ksize: int) -> float:
    return 0.0 if ksize <= 1 else 0.3 * (0.5 * (ksize - 1) - 1.0) + 0.8


def sep_filter(src: torch.Tensor, taps: Sequence[float], along_y: bool) -> torch.Tensor:
    """One pass of a 1-D filter with replicated borders, result clamped and rounded to uint8."""
    src = _prep(src)
    h, w, c = src.shape
    taps = np.asarray(taps, dtype=np.float32)
    r = len(taps) // 2
    if src.is_cuda:
        if len(taps) > 64:
            raise ValueError("filter taps are limited to 64")
        dst = torch.empty_like(src)
        buf = (ctypes.c_float * len(taps))(*[float(t) for t in taps])
        _launch("mmj_vis_sep_filter", _C.ptr(src), _C.ptr(dst), h, w, c, buf, r, int(along_y), _stream())
        return dst
    a = src.numpy().astype(np.float32)
    axis = 0 if along_y else 1
    n = a.shape[axis]
    acc = np.zeros_like(a)
    for k in range(-r, r + 1):
        idx = np.clip(np.arange(n) + k, 0, n - 1)
        acc += np.float32(taps[k + r]) * np.take(a, idx, axis=axis)
    return torch.from_numpy((np.clip(acc, 0, 255) + np.float32(0.5)).astype(np.uint8))


def gaussian_blur(src: torch.Tensor, kx: int, ky: int, sigma: float) -> torch.Tensor:
    sx = sigma if sigma > 0 else sigma_from_ksize(kx)
    sy = sigma if sigma > 0 else sigma_from_ksize(ky)
    tmp = sep_filter(src, gaussian_taps(kx, sx), along_y=False)
    return sep_filter(tmp, gaussian_taps(ky, sy), along_y=True)


# ---- 3x3 derivatives ---------------------------------------------------------------------------------
DERIV_SOBEL_X, DERIV_SOBEL_Y, DERIV_LAPLACE, DERIV_MAGNITUDE = 0, 1, 2, 3


def deriv3(gray: torch.Tensor, mode: int) -> torch.Tensor:
    gray = _prep(gray)
    h, w, c = gray.shape
    if c != 1:
        raise ValueError("derivative filters take a single-channel image")
    if gray.is_cuda:
        dst = torch.empty_like(gray)
        _launch("mmj_vis_deriv3", _C.ptr(gray), _C.ptr(dst), h, w, mode, _stream())
        return dst
    a = np.pad(gray.numpy()[..., 0].astype(np.int32), 1, mode="edge")
    s = lambda dy, dx: a[1 + dy:1 + dy + h, 1 + dx:1 + dx + w]
    gx = (s(-1, 1) + 2 * s(0, 1) + s(1, 1)) - (s(-1, -1) + 2 * s(0, -1) + s(1, -1))
    gy = (s(1, -1) + 2 * s(1, 0) + s(1, 1)) - (s(-1, -1) + 2 * s(-1, 0) + s(-1, 1))
    if mode == DERIV_SOBEL_X:
        v = np.abs(gx)
    elif mode == DERIV_SOBEL_Y:
        v = np.abs(gy)
    elif mode == DERIV_LAPLACE:
        v = np.abs(s(-1, 0) + s(0, -1) + s(0, 1) + s(1, 0) - 4 * s(0, 0))
    else:
        v = (np.sqrt((gx * gx + gy * gy).astype(np.float32)) + np.float32(0.5)).astype(np.int32)
    return torch.from_numpy(np.minimum(v, 255).astype(np.uint8)[..., None])


# ---- morphology --------------------------------------------------------------------------------------
def morph(src: torch.Tensor, ksize: int, dilate: bool) -> torch.Tensor:
    src = _prep(src)
    h, w, c = src.shape
    ksize = max(int(ksize), 1)
    if src.is_cuda:
        dst = torch.empty_like(src)
        _launch("mmj_vis_morph", _C.ptr(src), _C.ptr(dst), h, w, c, ksize, int(dilate), _stream())
        return dst
    r = ksize // 2
    a = src.numpy()
    pad_val = 0 if dilate else 255
    p = np.pad(a, ((r, r), (r, r), (0, 0)), mode="constant", constant_values=pad_val)
    out = np.full_like(a, pad_val)
    f = np.maximum if dilate else np.minimum
    for dy in range(2 * r + 1):
        for dx in range(2 * r + 1):
            out = f(out, p[dy:dy + h, dx:dx + w])
    return torch.from_numpy(out)


# ---- warps ------------------------------------------------------------------------------------------
def _border_index(v: np.ndarray, n: int, border: int):
    inside = (v >= 0) & (v < n)
    if border == BORDER_REPLICATE:
        return np.clip(v, 0, n - 1), np.ones_like(inside)
    if border == BORDER_REFLECT:
        if n == 1:
            return np.zeros_like(v), np.ones_like(inside)
        period = 2 * (n - 1)
        m = np.mod(v, period)
        return np.where(m < n, m, period - m), np.ones_like(inside)
    return np.where(inside, v, 0), inside


def warp(src: torch.Tensor, inv: Sequence[float], perspective: bool, border: int = 0, fill: int = 0) -> torch.Tensor:
    """Nearest-sample warp: output pixel (x, y) takes the source pixel at floor(inv @ [x, y, 1] + 0.5)."""
    src = _prep(src)
    h, w, c = src.shape
    inv = [float(v) for v in inv]
    if src.is_cuda:
        dst = torch.empty_like(src)
        buf = (ctypes.c_double * 9)(*inv)
        _launch("mmj_vis_warp", _C.ptr(src), _C.ptr(dst), h, w, c, buf, int(perspective), int(border),
                int(fill) & 255, _stream())
        return dst
    a = src.numpy()
    ys, xs = np.mgrid[0:h, 0:w].astype(np.float64)
    u = inv[0] * xs + inv[1] * ys + inv[2]
    v = inv[3] * xs + inv[4] * ys + inv[5]
    ok = np.ones((h, w), dtype=bool)
    if perspective:
        z = inv[6] * xs + inv[7] * ys + inv[8]
        ok = z != 0.0
        zs = np.where(ok, z, 1.0)
        u, v = u / zs, v / zs
    sx, inx = _border_index(np.floor(u + 0.5).astype(np.int64), w, border)
    sy, iny = _border_index(np.floor(v + 0.5).astype(np.int64), h, border)
    out = a[sy, sx]
    out = np.where((inx & iny)[..., None], out, np.uint8(int(fill) & 255))
    out = np.where(ok[..., None], out, np.uint8(0))
    return torch.from_numpy(np.ascontiguousarray(out.astype(np.uint8)))


# ---- histogram / LUT -----------------------------------------------------------------------------------
def histogram(src: torch.Tensor, channel: int = 0) -> torch.Tensor:
    """256-bin count of one channel (int64 tensor on the image's device)."""
    src = _prep(src)
    h, w, c = src.shape
    if src.is_cuda:
        bins = torch.zeros(256, dtype=torch.int32, device=src.device)
        _launch("mmj_vis_hist", _C.ptr(src), h * w, c, channel, _C.ptr(bins), _stream())
        return bins.to(torch.int64)
    return torch.from_numpy(np.bincount(src.numpy()[..., channel].reshape(-1), minlength=256).astype(np.int64))


def apply_lut(src: torch.Tensor, lut) -> torch.Tensor:
    src = _prep(src)
    lut = torch.as_tensor(lut, dtype=torch.uint8)
    if src.is_cuda:
        lut = lut.to(src.device).contiguous()
        dst = torch.empty_like(src)
        _launch("mmj_vis_lut", _C.ptr(src), _C.ptr(dst), src.numel(), _C.ptr(lut), _stream())
        return dst
    return torch.from_numpy(lut.numpy()[src.numpy()])


# ---- pointwise ---------------------------------------------------------------------------------------
OP_AND, OP_OR, OP_NOT, OP_WEIGHTED = 0, 1, 2, 3


def binary(a: torch.Tensor, b, op: int, alpha: float = 1.0, beta: float = 1.0, gamma: float = 0.0) -> torch.Tensor:
    a = _prep(a)
    if b is not None:
        b = _prep(b)
        if b.shape != a.shape:
            raise ValueError(f"image shapes differ: {tuple(a.shape)} vs {tuple(b.shape)}")
    if a.is_cuda:
        dst = torch.empty_like(a)
        _launch("mmj_vis_binary", _C.ptr(a), _C.ptr(b) if b is not None else None, _C.ptr(dst), a.numel(),
                op, float(alpha), float(beta), float(gamma), _stream())
        return dst
    x = a.numpy()
    y = b.numpy() if b is not None else np.zeros_like(x)
    if op == OP_AND:
        r = x & y
    elif op == OP_OR:
        r = x | y
    elif op == OP_NOT:
        r = ~x
    else:
        f = x.astype(np.float32) * np.float32(alpha) + y.astype(np.float32) * np.float32(beta) + np.float32(gamma)
        r = (np.clip(f, 0, 255) + np.float32(0.5)).astype(np.uint8)
    return torch.from_numpy(np.ascontiguousarray(r))


# ---- neighbourhood / region kernels (device tensors only; the transforms keep their host restatements) ----
def median(src: torch.Tensor, ksize: int) -> torch.Tensor:
    """k x k median with a replicated border (k odd, <= 9); ``src`` is a CUDA HWC uint8 tensor."""
    src = _prep(src)
    h, w, c = src.shape
    dst = torch.empty_like(src)
    _launch("mmj_vis_median", _C.ptr(src), _C.ptr(dst), h, w, c, int(ksize), _stream())
    return dst


def bilateral(src: torch.Tensor, radius: int, sigma_color: float, sigma_space: float) -> torch.Tensor:
    src = _prep(src)
    h, w, c = src.shape
    dst = torch.empty_like(src)
    sc2 = 2.0 * max(float(sigma_color), 1e-6) ** 2
    ss2 = 2.0 * max(float(sigma_space), 1e-6) ** 2
    _launch("mmj_vis_bilateral", _C.ptr(src), _C.ptr(dst), h, w, c, int(radius), sc2, ss2, _stream())
    return dst


def canny(gray: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Sobel + L1 magnitude + non-maximum suppression + hysteresis on a CUDA [H, W, 1] uint8 image."""
    gray = _prep(gray)
    h, w, _ = gray.shape
    cls = torch.empty((h, w), dtype=torch.uint8, device=gray.device)
    _launch("mmj_vis_canny_nms", _C.ptr(gray), _C.ptr(cls), h, w, int(lo), int(hi), _stream())
    changed = torch.zeros(1, dtype=torch.int32, device=gray.device)
    for _ in range(h + w):   # a path can wind through the tiles; in practice a handful of passes
        changed.zero_()
        _launch("mmj_vis_canny_hysteresis", _C.ptr(cls), h, w, _C.ptr(changed), _stream())
        if int(changed.item()) == 0:
            break
    out = torch.empty((h, w, 1), dtype=torch.uint8, device=gray.device)
    _launch("mmj_vis_canny_finish", _C.ptr(cls), _C.ptr(out), h * w, _stream())
    return out


def clahe_plane(plane: torch.Tensor, clip_limit: float, tile: int) -> torch.Tensor:
    """Contrast-limited adaptive equalisation of a CUDA [H, W] uint8 plane (tile grid ``tile`` x ``tile``)."""
    plane = plane.contiguous()
    h, w = plane.shape
    ty, tx = max(1, min(tile, h)), max(1, min(tile, w))
    ys = np.linspace(0, h, ty + 1).astype(np.int32)
    xs = np.linspace(0, w, tx + 1).astype(np.int32)
    cy = (ys[:-1] + ys[1:]) / 2.0
    cx = (xs[:-1] + xs[1:]) / 2.0
    fi = np.clip(np.interp(np.arange(h) + 0.5, cy, np.arange(ty)), 0, ty - 1).astype(np.float32)
    fj = np.clip(np.interp(np.arange(w) + 0.5, cx, np.arange(tx)), 0, tx - 1).astype(np.float32)
    dev = plane.device
    ys_d, xs_d = torch.from_numpy(ys).to(dev), torch.from_numpy(xs).to(dev)
    fi_d, fj_d = torch.from_numpy(fi).to(dev), torch.from_numpy(fj).to(dev)
    luts = torch.empty((ty * tx, 256), dtype=torch.float32, device=dev)
    _launch("mmj_vis_clahe_luts", _C.ptr(plane), w, _C.ptr(ys_d), _C.ptr(xs_d), ty, tx, float(clip_limit),
            _C.ptr(luts), _stream())
    out = torch.empty_like(plane)
    _launch("mmj_vis_clahe_apply", _C.ptr(plane), _C.ptr(out), h, w, _C.ptr(fi_d), _C.ptr(fj_d), ty, tx,
            _C.ptr(luts), _stream())
    return out


def connected_components(bw: torch.Tensor, connectivity: int = 4):
    """``(count, labels)``: int64 [H, W] labels 1..count in row-major order of each component's first pixel,
    0 for background; ``bw`` is a CUDA uint8 [H, W] or [H, W, C] tensor (channel 0 decides)."""
    if bw.dim() == 3:
        stride, (h, w) = bw.shape[2], bw.shape[:2]
    else:
        stride, (h, w) = 1, bw.shape
    bw = bw.contiguous()
    labels = torch.empty(h * w, dtype=torch.int32, device=bw.device)
    _launch("mmj_vis_cc_init", _C.ptr(bw), stride, _C.ptr(labels), h * w, _stream())
    changed = torch.zeros(1, dtype=torch.int32, device=bw.device)
    for _ in range(h * w):
        changed.zero_()
        _launch("mmj_vis_cc_pass", _C.ptr(labels), h, w, int(connectivity == 8), _C.ptr(changed), _stream())
        if int(changed.item()) == 0:
            break
    roots, inverse = torch.unique(labels, sorted=True, return_inverse=True)   # roots ascend = discovery order
    has_bg = bool(roots.numel() and roots[0].item() == 0)
    out = inverse.to(torch.int64) + (0 if has_bg else 1)
    return int(roots.numel() - (1 if has_bg else 0)), out.reshape(h, w)
