"""Hough transforms (legacy/src/momijo/vision/transforms/hough.mojo:109-484) over the non-zero
pixels of channel 0."""
from __future__ import annotations

import math
from typing import List, Tuple

import numpy as np

from ..image import Image


def _edge_points(img: Image):
    a = img.numpy()[..., 0]
    ys, xs = np.nonzero(a)
    return a.shape[0], a.shape[1], xs.astype(np.float64), ys.astype(np.float64)


def _accumulate(img: Image, rho: float, theta: float):
    h, w, xs, ys = _edge_points(img)
    rho = max(float(rho), 1e-6)
    n_theta = max(int(round(math.pi / max(float(theta), 1e-6))), 1)
    thetas = np.arange(n_theta) * (math.pi / n_theta)
    diag = math.hypot(h, w)
    n_rho = int(2 * diag / rho) + 2
    acc = np.zeros((n_rho, n_theta), dtype=np.int32)
    if len(xs):
        r = xs[:, None] * np.cos(thetas)[None] + ys[:, None] * np.sin(thetas)[None]
        ri = np.round((r + diag) / rho).astype(np.int64)
        np.add.at(acc, (ri.reshape(-1), np.tile(np.arange(n_theta), len(xs))), 1)
    return acc, thetas, diag, rho, h, w


def hough_lines(img: Image, rho: float, theta: float, thresh: int) -> List[Tuple[int, int, int, int]]:
    """Infinite lines clipped to the image, as ``(x0, y0, x1, y1)``, strongest first."""
    acc, thetas, diag, rho, h, w = _accumulate(img, rho, theta)
    out = []
    cand = np.argwhere(acc >= max(int(thresh), 1))
    cand = sorted(cand.tolist(), key=lambda p: -acc[p[0], p[1]])
    for ri, ti in cand:
        nb = acc[max(ri - 1, 0):ri + 2, max(ti - 1, 0):ti + 2]
        if acc[ri, ti] < nb.max():
            continue
        r, t = ri * rho - diag, thetas[ti]
        c, s = math.cos(t), math.sin(t)
        x0, y0 = c * r, s * r
        L = diag
        out.append((int(round(x0 - L * s)), int(round(y0 + L * c)), int(round(x0 + L * s)), int(round(y0 - L * c))))
    return out


def hough_lines_p(img: Image, rho: float, theta: float, threshold: int, min_len: int = 0, max_gap: int = 0):
    """Segments supported by edge pixels: each accumulator peak is walked along its line, splitting
    at gaps longer than ``max_gap`` and dropping pieces shorter than ``min_len``."""
    a = img.numpy()[..., 0] != 0
    h, w = a.shape
    segs = []
    for x0, y0, x1, y1 in hough_lines(img, rho, theta, threshold):
        n = int(max(abs(x1 - x0), abs(y1 - y0))) + 1
        xs = np.round(np.linspace(x0, x1, n)).astype(int)
        ys = np.round(np.linspace(y0, y1, n)).astype(int)
        start, last, gap = None, None, 0
        for x, y in zip(xs, ys):
            on = 0 <= x < w and 0 <= y < h and a[max(y - 1, 0):y + 2, max(x - 1, 0):x + 2].any()
            if on:
                if start is None:
                    start = (x, y)
                last, gap = (x, y), 0
            elif start is not None:
                gap += 1
                if gap > max_gap:
                    if math.hypot(last[0] - start[0], last[1] - start[1]) >= min_len:
                        segs.append((int(start[0]), int(start[1]), int(last[0]), int(last[1])))
                    start = None
        if start is not None and math.hypot(last[0] - start[0], last[1] - start[1]) >= min_len:
            segs.append((int(start[0]), int(start[1]), int(last[0]), int(last[1])))
    return segs


def hough_circles(img: Image, *args, dp: float = 1.0, min_dist=50, param1: float = 100.0, param2: float = 30.0,
                  min_r: int = 0, max_r: int = 0, method: int = 0) -> List[Tuple[int, int, int]]:
    """Centres and radii ``(x, y, r)``. Positional forms: ``(method, dp, minDist)`` or
    ``(dp, min_dist, param1, param2, min_r, max_r)``."""
    if len(args) == 3:
        method, dp, min_dist = args
    elif len(args) >= 1:
        names = ["dp", "min_dist", "param1", "param2", "min_r", "max_r"]
        vals = dict(zip(names, args))
        dp, min_dist = vals.get("dp", dp), vals.get("min_dist", min_dist)
        param1, param2 = vals.get("param1", param1), vals.get("param2", param2)
        min_r, max_r = vals.get("min_r", min_r), vals.get("max_r", max_r)
    from .filter import canny
    g = img if img.channels() == 1 else None
    edges = canny(img, int(param1 / 2), int(param1)) if img.numpy().max() > 1 and len(np.unique(img.numpy())) > 2 else img
    a = edges.numpy()[..., 0] != 0
    h, w = a.shape
    ys, xs = np.nonzero(a)
    if len(xs) == 0:
        return []
    max_r = int(max_r) if max_r > 0 else min(h, w) // 2
    min_r = max(int(min_r), 1)
    angles = np.linspace(0, 2 * math.pi, 64, endpoint=False)
    found = []
    for r in range(min_r, max_r + 1):
        acc = np.zeros((h, w), dtype=np.int32)
        cx = np.round(xs[:, None] - r * np.cos(angles)[None]).astype(int).reshape(-1)
        cy = np.round(ys[:, None] - r * np.sin(angles)[None]).astype(int).reshape(-1)
        ok = (cx >= 0) & (cx < w) & (cy >= 0) & (cy < h)
        np.add.at(acc, (cy[ok], cx[ok]), 1)
        for y, x in np.argwhere(acc >= max(param2, 1)):
            found.append((int(acc[y, x]), int(x), int(y), r))
    found.sort(reverse=True)
    out = []
    md = float(min_dist)
    for _, x, y, r in found:
        if all(math.hypot(x - ox, y - oy) >= md for ox, oy, _ in out):
            out.append((x, y, r))
    return out
