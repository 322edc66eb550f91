"""Netpbm codecs: P5/P6 binary and P2/P3 text (legacy/src/momijo/vision/io/ppm.mojo)."""
from __future__ import annotations

import numpy as np


def _tokens(buf: bytes, pos: int, n: int):
    out = []
    while len(out) < n:
        while pos < len(buf) and buf[pos:pos + 1].isspace():
            pos += 1
        if buf[pos:pos + 1] == b"#":
            while pos < len(buf) and buf[pos:pos + 1] != b"\n":
                pos += 1
            continue
        start = pos
        while pos < len(buf) and not buf[pos:pos + 1].isspace():
            pos += 1
        out.append(buf[start:pos])
    return out, pos


def decode_ppm(buf: bytes) -> np.ndarray:
    magic = buf[:2]
    if magic not in (b"P2", b"P3", b"P5", b"P6"):
        raise ValueError("not a PGM/PPM file")
    (w, h, maxval), pos = _tokens(buf, 2, 3)
    w, h, maxval = int(w), int(h), int(maxval)
    c = 3 if magic in (b"P3", b"P6") else 1
    n = w * h * c
    if magic in (b"P5", b"P6"):
        pos += 1  # the single whitespace byte after maxval
        if maxval < 256:
            a = np.frombuffer(buf, dtype=np.uint8, count=n, offset=pos).astype(np.int64)
        else:
            a = np.frombuffer(buf, dtype=">u2", count=n, offset=pos).astype(np.int64)
    else:
        toks, _ = _tokens(buf, pos, n)
        a = np.array([int(t) for t in toks], dtype=np.int64)
    if maxval != 255:
        a = (a * 255 + maxval // 2) // max(maxval, 1)
    return a.astype(np.uint8).reshape(h, w, c)


def encode_ppm(a: np.ndarray) -> bytes:
    if a.ndim == 2:
        a = a[..., None]
    h, w, c = a.shape
    if c == 1:
        return b"P5\n%d %d\n255\n" % (w, h) + np.ascontiguousarray(a).tobytes()
    return b"P6\n%d %d\n255\n" % (w, h) + np.ascontiguousarray(a[..., :3]).tobytes()
