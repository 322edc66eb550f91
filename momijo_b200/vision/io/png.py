"""PNG codec. The reference carries its own inflate, unfilter and encoder in Mojo
(legacy/src/momijo/vision/io/inflate.mojo, unfilter.mojo, decode_png.mojo, encode_png.mojo); here the
deflate stream goes through zlib and the scanline filters are restated with numpy.

Reader: non-interlaced, bit depths 1/2/4/8/16, colour types 0 (grey), 2 (RGB), 3 (palette, tRNS
honoured), 4 (grey+alpha), 6 (RGBA). Writer: 8-bit grey, grey+alpha, RGB or RGBA, filter type chosen per
row by the minimum-sum-of-absolute-differences heuristic among None/Sub/Up."""
from __future__ import annotations

import struct
import zlib

import numpy as np

_SIG = b"\x89PNG\r\n\x1a\n"


def _unfilter(raw: bytes, h: int, stride: int, bpp: int) -> np.ndarray:
    out = np.zeros((h, stride), dtype=np.uint8)
    prev = np.zeros(stride, dtype=np.int32)
    pos = 0
    for y in range(h):
        ft = raw[pos]
        line = np.frombuffer(raw, dtype=np.uint8, count=stride, offset=pos + 1).astype(np.int32)
        pos += stride + 1
        if ft == 0:
            cur = line
        elif ft == 2:
            cur = (line + prev) & 255
        elif ft == 1:
            cur = line.copy()
            for i in range(bpp, stride):
                cur[i] = (cur[i] + cur[i - bpp]) & 255
        elif ft == 3:
            cur = line.copy()
            for i in range(stride):
                left = cur[i - bpp] if i >= bpp else 0
                cur[i] = (cur[i] + ((left + prev[i]) >> 1)) & 255
        elif ft == 4:
            cur = line.copy()
            for i in range(stride):
                a = cur[i - bpp] if i >= bpp else 0
                b = prev[i]
                c = prev[i - bpp] if i >= bpp else 0
                p = a + b - c
                pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
                pred = a if (pa <= pb and pa <= pc) else (b if pb <= pc else c)
                cur[i] = (cur[i] + pred) & 255
        else:
            raise ValueError(f"bad PNG filter type {ft}")
        out[y] = cur
        prev = cur
    return out


def decode_png(buf: bytes) -> np.ndarray:
    if buf[:8] != _SIG:
        raise ValueError("not a PNG file")
    pos = 8
    idat = []
    plte = trns = None
    hdr = None
    while pos + 8 <= len(buf):
        n, typ = struct.unpack(">I4s", buf[pos:pos + 8])
        data = buf[pos + 8:pos + 8 + n]
        pos += 12 + n
        if typ == b"IHDR":
            hdr = struct.unpack(">IIBBBBB", data)
        elif typ == b"PLTE":
            plte = np.frombuffer(data, dtype=np.uint8).reshape(-1, 3)
        elif typ == b"tRNS":
            trns = np.frombuffer(data, dtype=np.uint8)
        elif typ == b"IDAT":
            idat.append(data)
        elif typ == b"IEND":
            break
    if hdr is None:
        raise ValueError("PNG without IHDR")
    w, h, depth, ctype, _, _, interlace = hdr
    if interlace:
        raise ValueError("interlaced PNG is not supported")
    chans = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}[ctype]
    bits = depth * chans
    stride = (w * bits + 7) // 8
    bpp = max(bits // 8, 1)
    rows = _unfilter(zlib.decompress(b"".join(idat)), h, stride, bpp)
    if depth == 8:
        px = rows.reshape(h, w, chans)
    elif depth == 16:
        px = rows.reshape(h, w, chans, 2)[..., 0]
    else:
        bitsarr = np.unpackbits(rows, axis=1)[:, :w * depth * chans].reshape(h, w * chans, depth)
        vals = (bitsarr * (1 << np.arange(depth - 1, -1, -1))).sum(-1)
        px = vals.reshape(h, w, chans)
        if ctype != 3:
            px = (px * 255) // ((1 << depth) - 1)
        px = px.astype(np.uint8)
    if ctype == 3:
        if plte is None:
            raise ValueError("palette PNG without PLTE")
        idx = px[..., 0].astype(np.int64)
        rgb = plte[np.minimum(idx, len(plte) - 1)]
        if trns is not None:
            alpha = np.full(256, 255, dtype=np.uint8)
            alpha[:len(trns)] = trns
            px = np.concatenate([rgb, alpha[idx][..., None]], -1)
        else:
            px = rgb
    return np.ascontiguousarray(px.astype(np.uint8))


def _chunk(typ: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + typ + data + struct.pack(">I", zlib.crc32(typ + data) & 0xFFFFFFFF)


def encode_png(a: np.ndarray, level: int = 6) -> bytes:
    if a.ndim == 2:
        a = a[..., None]
    a = np.ascontiguousarray(a.astype(np.uint8))
    h, w, c = a.shape
    ctype = {1: 0, 2: 4, 3: 2, 4: 6}[c]
    rows = a.reshape(h, w * c).astype(np.int16)
    sub = rows.copy()
    sub[:, c:] -= rows[:, :-c]
    up = rows.copy()
    up[1:] -= rows[:-1]
    cands = [rows & 255, sub & 255, up & 255]
    cost = [np.minimum(x, 256 - x).sum(1) for x in cands]
    choice = np.argmin(np.stack(cost, 0), 0)
    out = bytearray()
    for y in range(h):
        k = int(choice[y])
        out.append(k)
        out += cands[k][y].astype(np.uint8).tobytes()
    ihdr = struct.pack(">IIBBBBB", w, h, 8, ctype, 0, 0, 0)
    return _SIG + _chunk(b"IHDR", ihdr) + _chunk(b"IDAT", zlib.compress(bytes(out), level)) + _chunk(b"IEND", b"")
