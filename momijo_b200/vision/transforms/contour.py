"""Contours (legacy/src/momijo/vision/transforms/contour.mojo:125-580): border following over the
non-zero pixels of channel 0; points are ``(x, y)``."""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import numpy as np

from ..image import Image


def is_on_u8(img: Image, x: int, y: int, thresh: int = 0) -> bool:
    return 0 <= x < img.width() and 0 <= y < img.height() and img.get_u8(y, x, 0) > thresh


_DIRS = [(1, 0), (1, 1), (0, 1), (-1, 1), (-1, 0), (-1, -1), (0, -1), (1, -1)]  # clockwise from east (y down)


def _trace(fg: np.ndarray, sx: int, sy: int) -> List[Tuple[int, int]]:
    h, w = fg.shape
    on = lambda x, y: 0 <= x < w and 0 <= y < h and fg[y, x]
    pts = [(sx, sy)]
    x, y, d = sx, sy, 6  # arrived "from the west": start searching from north
    first_move = None
    for _ in range(4 * h * w + 8):
        found = False
        for k in range(8):
            nd = (d + k) % 8
            nx, ny = x + _DIRS[nd][0], y + _DIRS[nd][1]
            if on(nx, ny):
                move = (x, y, nd)
                if first_move is None:
                    first_move = move
                elif move == first_move:
                    return pts[:-1] if len(pts) > 1 and pts[-1] == pts[0] else pts
                x, y = nx, ny
                pts.append((x, y))
                d = (nd + 5) % 8  # back up two steps counter-clockwise from the arrival direction
                found = True
                break
        if not found:
            return pts
    return pts


def find_contours(img: Image, external_only: bool = False) -> List[List[Tuple[int, int]]]:
    a = img.numpy()[..., 0]
    fg = a != 0
    h, w = fg.shape
    from .segmentation import connected_components
    _, lab = connected_components(fg.astype(np.uint8), 8)
    lab = np.asarray(lab)
    contours, seen = [], set()
    for y in range(h):
        for x in range(w):
            l = lab[y, x]
            if l and l not in seen and (x == 0 or not fg[y, x - 1]):
                seen.add(l)
                contours.append(_trace(fg, x, y))
    if not external_only:
        # hole borders: background components that do not touch the image border
        _, hl = connected_components((~fg).astype(np.uint8), 4)
        hl = np.asarray(hl)
        border = set(hl[0, :]) | set(hl[-1, :]) | set(hl[:, 0]) | set(hl[:, -1])
        done = set()
        for y in range(h):
            for x in range(w):
                l = hl[y, x]
                if l and l not in border and l not in done:
                    done.add(l)
                    contours.append(_trace(fg, x - 1, y) if x > 0 and fg[y, x - 1] else _trace(fg, x, y - 1))
    return contours


def get_contour(contours, idx: int):
    return contours[idx] if 0 <= idx < len(contours) else []


def len_contours(cs) -> int:
    return len(cs)


def bounding_rect(contour) -> Tuple[int, int, int, int]:
    if not contour:
        return (0, 0, 0, 0)
    xs = [p[0] for p in contour]
    ys = [p[1] for p in contour]
    return (min(xs), min(ys), max(xs) - min(xs) + 1, max(ys) - min(ys) + 1)


def contour_area(contour) -> float:
    n = len(contour)
    if n < 3:
        return 0.0
    s = 0.0
    for i in range(n):
        x0, y0 = contour[i]
        x1, y1 = contour[(i + 1) % n]
        s += x0 * y1 - x1 * y0
    return abs(s) * 0.5


def arc_length(points, closed: bool = False) -> float:
    pts = list(points)
    if pts and not isinstance(pts[0], (tuple, list)):
        pts = [(pts[i], pts[i + 1]) for i in range(0, len(pts) - 1, 2)]
    n = len(pts)
    if n < 2:
        return 0.0
    total = sum(math.hypot(pts[i + 1][0] - pts[i][0], pts[i + 1][1] - pts[i][1]) for i in range(n - 1))
    if closed:
        total += math.hypot(pts[0][0] - pts[-1][0], pts[0][1] - pts[-1][1])
    return float(total)
