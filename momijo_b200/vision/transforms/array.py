"""Array-style helpers and the ORB-like detector / Hamming matcher
(legacy/src/momijo/vision/transforms/array.mojo:54-440, features.mojo:57-210)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from ..image import Image
from .. import kernels as K

class Descriptor(list):
    """A list of binary rows (ORB-like), each a list of 32 ints 0..255
    (legacy/src/momijo/vision/transforms/features.mojo:43-54)."""

    @property
    def rows(self):
        return self

    @staticmethod
    def null() -> "Descriptor":
        return Descriptor()


def zeros(*args, dtype=None) -> Image:
    """``zeros((h, w, c), dtype)`` or ``zeros(h, w, c, dtype)``."""
    if args and isinstance(args[0], (tuple, list)):
        h, w, c = args[0]
    else:
        h, w, c = args[:3]
    return Image.new_hwc_u8(h, w, c, 0)


def full(*args) -> Image:
    if isinstance(args[0], (tuple, list)):
        (h, w, c), value = args[0], args[1]
    else:
        h, w, c, value = args
    return Image.new_hwc_u8(h, w, c, value)


def full_like(img: Image, value: int) -> Image:
    return Image(torch.full_like(img.data, int(value) & 255), img.meta().copy())


def fill(img: Image, color: Sequence[int]) -> Image:
    c = img.channels()
    vals = [int(color[min(k, len(color) - 1)]) & 255 for k in range(c)]
    img.data[...] = torch.tensor(vals, dtype=torch.uint8, device=img.device)
    return img


def fill_scalar(img: Image, value: int) -> Image:
    img.data.fill_(int(value) & 255)
    return img


def fill3(img: Image, b: int, g: int, r: int) -> Image:
    return fill(img, [b, g, r])


def add_weighted(a: Image, alpha: float, b: Image, beta: float, gamma: float) -> Image:
    return Image(K.binary(a.data, b.data, K.OP_WEIGHTED, alpha, beta, gamma), a.meta().copy())


def abs_u8(img: Image) -> Image:
    return img.clone()  # uint8 is its own absolute value


def copy_to(src: Image, dst: Image) -> None:
    h, w, c = min(src.h, dst.h), min(src.w, dst.w), min(src.c, dst.c)
    dst.data[:h, :w, :c] = src.data[:h, :w, :c].to(dst.device)


def top_k_indices(k: int) -> List[int]:
    return list(range(max(int(k), 0)))


# ---- features ------------------------------------------------------------------------------------------
def _brief_pattern(n_bits: int = 256, patch: int = 15, seed: int = 0x9E3779B9):
    state = seed
    pts = []
    for _ in range(n_bits * 4):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        pts.append(int((state >> 16) % (2 * patch + 1)) - patch)
    return np.array(pts, dtype=np.int64).reshape(n_bits, 4)


_PATTERN = _brief_pattern()


def orb_detect_and_compute(img: Image, n_features: int = 500):
    """FAST-9-style corners ranked by a Harris-like score, with 256-bit BRIEF descriptors.
    Returns ``(keypoints, descriptors)``: ``[(x, y, score)]`` and a list of 32-byte rows."""
    d = img.ensure_packed_hwc_u8().data
    g = (d if d.shape[2] == 1 else K.to_gray(d, bgr=True)).cpu().numpy()[..., 0].astype(np.int32)
    h, w = g.shape
    m = 16
    if h <= 2 * m or w <= 2 * m:
        return [], []
    circle = [(0, -3), (1, -3), (2, -2), (3, -1), (3, 0), (3, 1), (2, 2), (1, 3), (0, 3), (-1, 3), (-2, 2),
              (-3, 1), (-3, 0), (-3, -1), (-2, -2), (-1, -3)]
    core = g[m:h - m, m:w - m]
    t = 20
    ring = np.stack([g[m + dy:h - m + dy, m + dx:w - m + dx] for dx, dy in circle], 0)
    brighter = ring > core + t
    darker = ring < core - t

    def has_run(b):
        bb = np.concatenate([b, b[:8]], 0).astype(np.int32)
        run = np.zeros(b.shape[1:], dtype=np.int32)
        best = np.zeros_like(run)
        for i in range(bb.shape[0]):
            run = np.where(bb[i] > 0, run + 1, 0)
            best = np.maximum(best, run)
        return best >= 9

    corners = has_run(brighter) | has_run(darker)
    score = np.abs(ring - core).sum(0).astype(np.float32)
    score = np.where(corners, score, 0)
    # 3x3 non-maximum suppression
    sp = np.pad(score, 1)
    hh, ww = score.shape
    nb = np.max(np.stack([sp[dy:dy + hh, dx:dx + ww] for dy in range(3) for dx in range(3)], 0), 0)
    ys, xs = np.nonzero((score > 0) & (score >= nb))
    order = np.argsort(-score[ys, xs], kind="stable")[:max(int(n_features), 0)]
    blur = K.gaussian_blur(torch.from_numpy(g.astype(np.uint8)[..., None]), 5, 5, 0.0).numpy()[..., 0].astype(np.int32)
    kps, des = [], []
    for i in order:
        y, x = int(ys[i]) + m, int(xs[i]) + m
        a = blur[y + _PATTERN[:, 1], x + _PATTERN[:, 0]]
        b = blur[y + _PATTERN[:, 3], x + _PATTERN[:, 2]]
        bits = (a < b).astype(np.uint8)
        des.append([int(v) for v in np.packbits(bits)])
        kps.append((x, y, float(score[ys[i], xs[i]])))
    return kps, des


def len_keypoints(kps) -> int:
    return len(kps)


def keypoint_xy(kps, i: int) -> Tuple[int, int]:
    return int(kps[i][0]), int(kps[i][1])


def valid_descriptors(des) -> bool:
    return des is not None and len(des) > 0 and len(des[0]) > 0


_POP = np.array([bin(i).count("1") for i in range(256)], dtype=np.int32)


def bf_match_hamming(a, b, cross_check: bool = True) -> List[Tuple[int, int, int]]:
    """Brute-force matches ``(query index, train index, Hamming distance)``, sorted by distance."""
    if not valid_descriptors(a) or not valid_descriptors(b):
        return []
    A = np.asarray(a, dtype=np.uint8)
    B = np.asarray(b, dtype=np.uint8)
    dist = _POP[A[:, None, :] ^ B[None, :, :]].sum(-1)
    best_b = dist.argmin(1)
    out = []
    if cross_check:
        best_a = dist.argmin(0)
        for i, j in enumerate(best_b):
            if best_a[j] == i:
                out.append((i, int(j), int(dist[i, j])))
    else:
        out = [(i, int(j), int(dist[i, j])) for i, j in enumerate(best_b)]
    out.sort(key=lambda m: m[2])
    return out


def top_k_matches(matches, k: int):
    return sorted(matches, key=lambda m: m[2])[:max(int(k), 0)]


def to_int_triples(ms):
    return [(int(a), int(b), int(c)) for a, b, c in ms]
