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


# ---- the reference's byte-level PNG API (legacy/src/momijo/vision/io/png_decoder.mojo:12-120,
# legacy/src/momijo/vision/io/decode_png.mojo:162-262, legacy/src/momijo/vision/io/unfilter.mojo:33-110,
# legacy/src/momijo/vision/io/encode_png.mojo:760-810). Buffers are bytes-like objects or lists of ints;
# results that were ``List[UInt8]`` there are ``bytes`` here. "ptr + offset" arguments became (buffer, offset).
from dataclasses import dataclass  # noqa: E402


def read_be_u32(buf, off: int = 0) -> int:
    return int.from_bytes(bytes(buf[off:off + 4]), "big")


def is_png_magic(buf, off: int = 0) -> bool:
    return bytes(buf[off:off + 8]) == _SIG


@dataclass
class PNGChunk:
    length: int
    chunk_type: tuple
    data: bytes          # the reference keeps a pointer into the file buffer
    crc: int

    @property
    def type_str(self) -> str:
        return bytes(self.chunk_type).decode("latin-1")


def parse_chunk(buf, off: int = 0) -> PNGChunk:
    """Chunk starting at ``off`` (no CRC verification here)."""
    b = bytes(buf)
    n = read_be_u32(b, off)
    return PNGChunk(n, tuple(b[off + 4:off + 8]), b[off + 8:off + 8 + n], read_be_u32(b, off + 8 + n))


@dataclass
class PNGHeader:
    width: int
    height: int
    bit_depth: int
    color_type: int
    compression: int
    filter: int
    interlace: int


def parse_ihdr(data, off: int = 0) -> PNGHeader:
    b = bytes(data)
    return PNGHeader(read_be_u32(b, off), read_be_u32(b, off + 4), b[off + 8], b[off + 9], b[off + 10], b[off + 11],
                     b[off + 12])


def read_png_header_only(file_data, length: int = None):
    """(found, header) from the IHDR chunk without touching the pixel data."""
    b = bytes(file_data)
    length = len(b) if length is None else min(length, len(b))
    empty = PNGHeader(0, 0, 0, 0, 0, 0, 0)
    if length < 8 or not is_png_magic(b):
        return False, empty
    cur = 8
    while cur + 12 <= length:
        ch = parse_chunk(b, cur)
        if ch.type_str == "IHDR":
            return True, parse_ihdr(ch.data)
        if ch.type_str == "IEND":
            break
        cur += 12 + ch.length
    return False, empty


def parse_png_header(data):
    """(ok, width, height, bit_depth, color_type, PLTE bytes, tRNS bytes)."""
    b = bytes(data)
    ok, h = read_png_header_only(b)
    if not ok:
        return False, 0, 0, 0, 0, b"", b""
    plte = trns = b""
    cur = 8
    while cur + 12 <= len(b):
        ch = parse_chunk(b, cur)
        if ch.type_str == "PLTE":
            plte = ch.data
        elif ch.type_str == "tRNS":
            trns = ch.data
        elif ch.type_str == "IEND":
            break
        cur += 12 + ch.length
    return True, h.width, h.height, h.bit_depth, h.color_type, plte, trns


def decode_png_bytes(data):
    """(ok, width, height, channels, packed HWC uint8 bytes); 16-bit files keep their high bytes."""
    try:
        a = decode_png(bytes(data))
    except Exception:   # any malformed input is reported through ``ok``
        return False, 0, 0, 0, b""
    return True, a.shape[1], a.shape[0], a.shape[2], a.tobytes()


def decode_png_bytes_u16(data):
    """(ok, width, height, channels, list of 16-bit samples): 16-bit files at full precision, 8-bit files
    scaled by 257 (so that 255 maps to 65535)."""
    b = bytes(data)
    ok, hdr = read_png_header_only(b)
    if not ok:
        return False, 0, 0, 0, []
    if hdr.bit_depth != 16:
        ok, w, h, c, px = decode_png_bytes(b)
        return (True, w, h, c, [v * 257 for v in px]) if ok else (False, 0, 0, 0, [])
    try:
        idat, cur = [], 8
        while cur + 12 <= len(b):
            ch = parse_chunk(b, cur)
            if ch.type_str == "IDAT":
                idat.append(ch.data)
            cur += 12 + ch.length
        chans = {0: 1, 2: 3, 4: 2, 6: 4}[hdr.color_type]
        stride = hdr.width * chans * 2
        rows = _unfilter(zlib.decompress(b"".join(idat)), hdr.height, stride, chans * 2)
        vals = rows.reshape(hdr.height, hdr.width * chans, 2).astype(np.uint16)
        return True, hdr.width, hdr.height, chans, ((vals[..., 0] << 8) | vals[..., 1]).reshape(-1).tolist()
    except Exception:
        return False, 0, 0, 0, []


def png_unfilter(width: int, height: int, channels: int, data, bit_depth: int = 8):
    """Undo the per-row filters of an inflated scan: (ok, bytes without the filter-type bytes)."""
    if width <= 0 or height <= 0 or channels <= 0 or bit_depth not in (1, 2, 4, 8, 16):
        return False, b""
    bits = channels * bit_depth
    stride = (width * bits + 7) // 8
    raw = bytes(data)
    if len(raw) < height * (stride + 1):
        return False, b""
    try:
        return True, _unfilter(raw, height, stride, max((bits + 7) // 8, 1)).tobytes()
    except ValueError:
        return False, b""


def png_from_hwc_u8(width: int, height: int, channels: int, data, interlace: int = 0, compress: int = 0,
                    filter_mode: int = 0, palette_mode: int = 0, max_colors: int = 256, bit_depth_out: int = 8):
    """(ok, PNG file bytes) for packed HWC uint8 pixels. ``compress`` 0 stores, 1 uses fixed and 2 dynamic
    Huffman codes; ``filter_mode`` 0 writes unfiltered rows and a negative value picks a filter per row.
    Interlacing, palettes and 16-bit output are not produced: those arguments must keep their defaults."""
    raw = bytes(data)
    if width <= 0 or height <= 0 or not 1 <= channels <= 4 or len(raw) != width * height * channels:
        return False, b""
    if interlace or palette_mode or bit_depth_out != 8:
        return False, b""
    from .deflate import zlib_deflate
    a = np.frombuffer(raw, dtype=np.uint8).reshape(height, width, channels)
    if filter_mode < 0:
        return True, encode_png(a, 9 if compress >= 2 else 1)
    ctype = {1: 0, 2: 4, 3: 2, 4: 6}[channels]
    scan = b"".join(b"\x00" + a[y].tobytes() for y in range(height))
    ihdr = struct.pack(">IIBBBBB", width, height, 8, ctype, 0, 0, 0)
    return True, _SIG + _chunk(b"IHDR", ihdr) + _chunk(b"IDAT", zlib_deflate(scan, compress)) + _chunk(b"IEND", b"")


def read_png_u16_raw(path: str):
    with open(path, "rb") as f:
        return decode_png_bytes_u16(f.read())


def debug_sample_rgb(H: int, W: int, C: int, buf, tag: str) -> None:
    """Print the corner and centre pixels of a packed HWC buffer."""
    if H == 0 or W == 0 or C == 0:
        print("[dbg]", tag, " empty")
        return
    b = bytes(buf)
    px = lambda y, x: tuple(b[(y * W + x) * C + k] for k in range(min(C, 3)))
    print("[dbg]", tag, "TL", px(0, 0), "TR", px(0, W - 1), "C", px(H // 2, W // 2), "BL", px(H - 1, 0),
          "BR", px(H - 1, W - 1))
