"""Drawing primitives on uint8 images (legacy/src/momijo/vision/transforms/draw.mojo). Colours are
per-channel sequences in the image's own channel order (BGR in the reference's examples). Drawing
happens in host memory; images in device memory are copied back afterwards."""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import numpy as np
import torch

from ..image import Image
from .glyphs import glyph_rows


def as_u8(xs: Sequence[int]) -> List[int]:
    return [max(0, min(255, int(v))) for v in xs]


def iabs(v: int) -> int:
    return -v if v < 0 else v


def bgr_u8(b: int, g: int, r: int) -> Tuple[int, int, int]:
    return tuple(as_u8((b, g, r)))


def Int32Mat(a: Sequence[Sequence[int]]) -> List[Tuple[int, int]]:
    return [(int(p[0]), int(p[1])) for p in a]


class _Canvas:
    """Numpy view of an image for the duration of one drawing call."""

    def __init__(self, img: Image):
        self.img = img
        self.on_device = img.data.is_cuda
        self.a = img.data.cpu().numpy() if self.on_device else img.data.numpy()

    def color(self, col):
        c = self.a.shape[2]
        col = list(col) if isinstance(col, (tuple, list)) else [col]
        return np.array([int(col[min(k, len(col) - 1)]) & 255 for k in range(c)], dtype=np.uint8)

    def dot(self, x, y, col, thickness=1):
        h, w = self.a.shape[:2]
        r = max(int(thickness), 1) // 2
        y0, y1, x0, x1 = max(y - r, 0), min(y + r, h - 1), max(x - r, 0), min(x + r, w - 1)
        if y0 <= y1 and x0 <= x1:
            self.a[y0:y1 + 1, x0:x1 + 1] = col

    def done(self):
        if self.on_device:
            self.img.data.copy_(torch.from_numpy(self.a))
        return self.img


def _line(cv: _Canvas, x1, y1, x2, y2, col, thickness):
    dx, dy = iabs(x2 - x1), -iabs(y2 - y1)
    sx, sy = (1 if x1 < x2 else -1), (1 if y1 < y2 else -1)
    err = dx + dy
    x, y = int(x1), int(y1)
    for _ in range(dx - dy + 2):
        cv.dot(x, y, col, thickness)
        if x == x2 and y == y2:
            break
        e2 = 2 * err
        if e2 >= dy:
            err += dy
            x += sx
        if e2 <= dx:
            err += dx
            y += sy


def line(img: Image, x1: int, y1: int, x2: int, y2: int, color, thickness: int = 1) -> Image:
    cv = _Canvas(img)
    _line(cv, int(x1), int(y1), int(x2), int(y2), cv.color(color), thickness)
    return cv.done()


def rectangle(img: Image, x1: int, y1: int, x2: int, y2: int, color, thickness: int = 1) -> Image:
    """Outline, or a filled box when ``thickness`` is negative."""
    cv = _Canvas(img)
    col = cv.color(color)
    xa, xb, ya, yb = min(x1, x2), max(x1, x2), min(y1, y2), max(y1, y2)
    if thickness < 0:
        h, w = cv.a.shape[:2]
        cv.a[max(ya, 0):min(yb, h - 1) + 1, max(xa, 0):min(xb, w - 1) + 1] = col
    else:
        for (p, q, r, s) in ((xa, ya, xb, ya), (xb, ya, xb, yb), (xb, yb, xa, yb), (xa, yb, xa, ya)):
            _line(cv, p, q, r, s, col, thickness)
    return cv.done()


rectangle_color = rectangle
rectangle_gray = rectangle


def _circle(cv: _Canvas, cx, cy, r, col, thickness):
    h, w = cv.a.shape[:2]
    r = max(int(r), 0)
    y0, y1, x0, x1 = max(cy - r - 1, 0), min(cy + r + 1, h - 1), max(cx - r - 1, 0), min(cx + r + 1, w - 1)
    if y0 > y1 or x0 > x1:
        return
    yy, xx = np.mgrid[y0:y1 + 1, x0:x1 + 1]
    d = np.sqrt((xx - cx) ** 2 + (yy - cy) ** 2)
    mask = d <= r + 0.5 if thickness < 0 else np.abs(d - r) <= max(thickness, 1) / 2.0
    cv.a[y0:y1 + 1, x0:x1 + 1][mask] = col


def circle(img: Image, cx: int, cy: int, r: int, color, thickness: int = 1) -> Image:
    cv = _Canvas(img)
    _circle(cv, int(cx), int(cy), r, cv.color(color), thickness)
    return cv.done()


def draw_circles(img: Image, circles, color=(0, 255, 0), thickness: int = 1, center_color=None) -> Image:
    cv = _Canvas(img)
    for x, y, r in circles:
        _circle(cv, int(x), int(y), int(r), cv.color(color), thickness)
        if center_color is not None:
            _circle(cv, int(x), int(y), 1, cv.color(center_color), -1)
    return cv.done()


def _points(pts):
    pts = list(pts)
    if pts and not isinstance(pts[0], (tuple, list)):
        pts = [(pts[i], pts[i + 1]) for i in range(0, len(pts) - 1, 2)]
    return [(int(p[0]), int(p[1])) for p in pts]


def fill_poly(img: Image, pts, color) -> Image:
    """Even-odd scanline fill of a polygon given as points, a flat list, or nested pairs."""
    cv = _Canvas(img)
    col = cv.color(color)
    P = _points(pts)
    if len(P) >= 3:
        h, w = cv.a.shape[:2]
        for y in range(max(min(p[1] for p in P), 0), min(max(p[1] for p in P), h - 1) + 1):
            xs = []
            for i in range(len(P)):
                (xa, ya), (xb, yb) = P[i], P[(i + 1) % len(P)]
                if ya == yb:
                    continue
                if min(ya, yb) <= y < max(ya, yb):
                    xs.append(xa + (y - ya) * (xb - xa) / (yb - ya))
            xs.sort()
            for i in range(0, len(xs) - 1, 2):
                a, b = max(int(math.ceil(xs[i])), 0), min(int(math.floor(xs[i + 1])), w - 1)
                if a <= b:
                    cv.a[y, a:b + 1] = col
        for i in range(len(P)):
            _line(cv, *P[i], *P[(i + 1) % len(P)], col, 1)
    return cv.done()


def arrowed_line(img: Image, x1: int, y1: int, x2: int, y2: int, color, thickness: int = 1,
                 tip_len: float = 0.1) -> Image:
    cv = _Canvas(img)
    col = cv.color(color)
    _line(cv, int(x1), int(y1), int(x2), int(y2), col, thickness)
    L = math.hypot(x2 - x1, y2 - y1) * tip_len
    ang = math.atan2(y1 - y2, x1 - x2)
    for s in (math.pi / 4, -math.pi / 4):
        _line(cv, int(x2), int(y2), int(round(x2 + L * math.cos(ang + s))), int(round(y2 + L * math.sin(ang + s))),
              col, thickness)
    return cv.done()


def draw_contours(img: Image, contours, idx: int = -1, color=(0, 255, 0), thickness: int = 1) -> Image:
    cv = _Canvas(img)
    col = cv.color(color)
    sel = range(len(contours)) if idx < 0 else [idx]
    for i in sel:
        c = contours[i]
        if thickness < 0:
            cv.done()
            fill_poly(img, c, color)
            cv = _Canvas(img)
            continue
        for j in range(len(c)):
            _line(cv, *map(int, c[j]), *map(int, c[(j + 1) % len(c)]), col, thickness)
    return cv.done()


def draw_lines_p(img: Image, lines, color=(0, 0, 255), thickness: int = 1) -> Image:
    cv = _Canvas(img)
    col = cv.color(color)
    for x1, y1, x2, y2 in lines:
        _line(cv, int(x1), int(y1), int(x2), int(y2), col, thickness)
    return cv.done()


def draw_matches(img1: Image, kps1, img2: Image, kps2, matches, color=(0, 255, 0), max_draw: int = 50) -> Image:
    """Side-by-side canvas with a line per match between keypoint positions."""
    h = max(img1.height(), img2.height())
    c = max(img1.channels(), img2.channels())
    out = Image.new_hwc_u8(h, img1.width() + img2.width(), c, 0)
    for src, x0 in ((img1, 0), (img2, img1.width())):
        d = src.data.cpu()
        if d.shape[2] != c:
            d = d[..., :1].expand(-1, -1, c)
        out.data[:src.height(), x0:x0 + src.width()] = d
    cv = _Canvas(out)
    col = cv.color(color)
    for qi, ti, _ in list(matches)[:max_draw]:
        xa, ya = int(kps1[qi][0]), int(kps1[qi][1])
        xb, yb = int(kps2[ti][0]) + img1.width(), int(kps2[ti][1])
        _line(cv, xa, ya, xb, yb, col, 1)
        _circle(cv, xa, ya, 3, col, 1)
        _circle(cv, xb, yb, 3, col, 1)
    return cv.done()


def put_text(img: Image, text: str, x: int, y: int, font: int = 0, scale: float = 1.0, color=(255, 255, 255),
             thickness: int = 1) -> Image:
    """5x7 bitmap font; ``(x, y)`` is the bottom-left corner of the first glyph."""
    cv = _Canvas(img)
    col = cv.color(color)
    s = max(int(round(scale)), 1)
    cx = int(x)
    for ch in str(text):
        rows = glyph_rows(ch)
        for ry, bits in enumerate(rows):
            for rx in range(5):
                if bits & (1 << (4 - rx)):
                    y0 = int(y) - (7 - ry) * s
                    x0 = cx + rx * s
                    h, w = cv.a.shape[:2]
                    ya, yb, xa, xb = max(y0, 0), min(y0 + s, h), max(x0, 0), min(x0 + s, w)
                    if ya < yb and xa < xb:
                        cv.a[ya:yb, xa:xb] = col
        cx += 6 * s
    return cv.done()


_PALETTE = [(0, 0, 0), (255, 0, 0), (0, 255, 0), (0, 0, 255), (255, 255, 0), (255, 0, 255), (0, 255, 255),
            (128, 128, 128), (255, 128, 0), (128, 0, 255)]


def label_to_color(lbl, num_labels: int = None):
    """BGR colour of a label id (draw.mojo:942-962), or, given a label matrix, a nested colour list."""
    if isinstance(lbl, (list, tuple, np.ndarray)):
        a = np.abs(np.asarray(lbl, dtype=np.int64)) % len(_PALETTE)
        return np.asarray(_PALETTE, dtype=np.uint8)[a].tolist()
    return _PALETTE[abs(int(lbl)) % len(_PALETTE)]


def label_to_color_image(labels, num_labels: int = None) -> Image:
    a = np.abs(np.asarray(labels, dtype=np.int64)) % len(_PALETTE)
    return Image(torch.from_numpy(np.asarray(_PALETTE, dtype=np.uint8)[a]))
