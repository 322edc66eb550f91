"""Baseline JPEG codec (sequential DCT, Huffman). The reference implements the same pieces in Mojo
(legacy/src/momijo/vision/io/jpeg_decoder.mojo, idct.mojo, huffman.mojo, jpeg_dct.mojo,
jpeg_quantize.mojo, jpeg_huffman_encode.mojo, jpeg_writer.mojo); here the block transforms are matrix
products in numpy and only the entropy coder walks bits.

Decoder: SOF0/SOF1 frames, 1 or 3 components, any sampling factors (chroma replicated up), restart
intervals. Encoder: YCbCr 4:4:4 (or grey), the Annex K tables scaled by ``quality``."""
from __future__ import annotations

import struct

import numpy as np

_ZZ = np.array([0, 1, 8, 16, 9, 2, 3, 10, 17, 24, 32, 25, 18, 11, 4, 5, 12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13,
                6, 7, 14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51, 58, 59, 52, 45,
                38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63])

_Q_LUM = np.array([16, 11, 10, 16, 24, 40, 51, 61, 12, 12, 14, 19, 26, 58, 60, 55, 14, 13, 16, 24, 40, 57, 69, 56,
                   14, 17, 22, 29, 51, 87, 80, 62, 18, 22, 37, 56, 68, 109, 103, 77, 24, 35, 55, 64, 81, 104, 113,
                   92, 49, 64, 78, 87, 103, 121, 120, 101, 72, 92, 95, 98, 112, 100, 103, 99])
_Q_CHR = np.array([17, 18, 24, 47, 99, 99, 99, 99, 18, 21, 26, 66, 99, 99, 99, 99, 24, 26, 56, 99, 99, 99, 99, 99,
                   47, 66, 99, 99, 99, 99, 99, 99] + [99] * 32)

_DC_LUM = ([0, 1, 5, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0], list(range(12)))
_DC_CHR = ([0, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0], list(range(12)))
_AC_LUM = ([0, 2, 1, 3, 3, 2, 4, 3, 5, 5, 4, 4, 0, 0, 1, 0x7D], list(bytes.fromhex(
    "01020300041105122131410613516107227114328191a1082342b1c11552d1f02433627282090a161718191a25262728292a3435"
    "363738393a434445464748494a535455565758595a636465666768696a737475767778797a838485868788898a92939495969798"
    "999aa2a3a4a5a6a7a8a9aab2b3b4b5b6b7b8b9bac2c3c4c5c6c7c8c9cad2d3d4d5d6d7d8d9dae1e2e3e4e5e6e7e8e9eaf1f2f3f4"
    "f5f6f7f8f9fa")))
_AC_CHR = ([0, 2, 1, 2, 4, 4, 3, 4, 7, 5, 4, 4, 0, 1, 2, 0x77], list(bytes.fromhex(
    "000102031104052131061241510761711322328108144291a1b1c109233352f0156272d10a162434e125f11718191a262728292a"
    "35363738393a434445464748494a535455565758595a636465666768696a737475767778797a82838485868788898a9293949596"
    "9798999aa2a3a4a5a6a7a8a9aab2b3b4b5b6b7b8b9bac2c3c4c5c6c7c8c9cad2d3d4d5d6d7d8d9dae2e3e4e5e6e7e8e9eaf2f3f4"
    "f5f6f7f8f9fa")))
for _b, _v in (_DC_LUM, _DC_CHR, _AC_LUM, _AC_CHR):
    assert sum(_b) == len(_v)


def _dct_matrix() -> np.ndarray:
    k = np.arange(8)[:, None]
    n = np.arange(8)[None, :]
    m = np.cos((2 * n + 1) * k * np.pi / 16.0) * 0.5
    m[0] *= 1.0 / np.sqrt(2.0)
    return m


_D = _dct_matrix()


def _codes(bits, vals):
    """Canonical Huffman codes: symbol -> (code, length)."""
    table, code, k = {}, 0, 0
    for length in range(1, 17):
        for _ in range(bits[length - 1]):
            table[vals[k]] = (code, length)
            code += 1
            k += 1
        code <<= 1
    return table


# ---- decoder ---------------------------------------------------------------------------------------------
class _Bits:
    def __init__(self, data: bytes, pos: int):
        self.d, self.p, self.acc, self.n = data, pos, 0, 0

    def _fill(self):
        while self.n <= 24:
            if self.p >= len(self.d):
                b = 0
            else:
                b = self.d[self.p]
                if b == 0xFF:
                    nxt = self.d[self.p + 1] if self.p + 1 < len(self.d) else 0
                    if nxt == 0:
                        self.p += 2
                    else:
                        b = 0  # a marker: feed zeros, leave the position on it
                        self.acc = (self.acc << 8) | b
                        self.n += 8
                        continue
                else:
                    self.p += 1
            self.acc = (self.acc << 8) | b
            self.n += 8

    def get(self, k: int) -> int:
        if k == 0:
            return 0
        if self.n < k:
            self._fill()
        self.n -= k
        return (self.acc >> self.n) & ((1 << k) - 1)

    def reset(self):
        self.acc, self.n = 0, 0
        # skip to just after the RSTn marker
        while self.p + 1 < len(self.d) and not (self.d[self.p] == 0xFF and 0xD0 <= self.d[self.p + 1] <= 0xD7):
            self.p += 1
        self.p += 2


def _decode_tables(bits, vals):
    """(mincode, maxcode, valptr) per length for the bit-serial decode."""
    look, code, k = {}, 0, 0
    for length in range(1, 17):
        for _ in range(bits[length - 1]):
            look[(length, code)] = vals[k]
            code += 1
            k += 1
        code <<= 1
    return look


def _huff(br: _Bits, look) -> int:
    code = 0
    for length in range(1, 17):
        code = (code << 1) | br.get(1)
        s = look.get((length, code))
        if s is not None:
            return s
    raise ValueError("corrupt JPEG entropy data")


def _extend(v: int, t: int) -> int:
    return v if t == 0 or v >= (1 << (t - 1)) else v - (1 << t) + 1


def decode_jpeg(buf: bytes) -> np.ndarray:
    if buf[:2] != b"\xff\xd8":
        raise ValueError("not a JPEG file")
    pos = 2
    qt, hdc, hac = {}, {}, {}
    frame = None
    restart = 0
    while pos < len(buf):
        if buf[pos] != 0xFF:
            pos += 1
            continue
        m = buf[pos + 1]
        pos += 2
        if m in (0xD8, 0x01) or 0xD0 <= m <= 0xD7:
            continue
        if m == 0xD9:
            break
        n = struct.unpack(">H", buf[pos:pos + 2])[0]
        seg = buf[pos + 2:pos + n]
        if m == 0xDB:
            i = 0
            while i < len(seg):
                pq, tq = seg[i] >> 4, seg[i] & 15
                i += 1
                if pq:
                    t = np.frombuffer(seg, dtype=">u2", count=64, offset=i).astype(np.int32)
                    i += 128
                else:
                    t = np.frombuffer(seg, dtype=np.uint8, count=64, offset=i).astype(np.int32)
                    i += 64
                q = np.zeros(64, dtype=np.int32)
                q[_ZZ] = t
                qt[tq] = q.reshape(8, 8)
        elif m == 0xC4:
            i = 0
            while i < len(seg):
                tc, th = seg[i] >> 4, seg[i] & 15
                bits = list(seg[i + 1:i + 17])
                cnt = sum(bits)
                vals = list(seg[i + 17:i + 17 + cnt])
                i += 17 + cnt
                (hac if tc else hdc)[th] = _decode_tables(bits, vals)
        elif m in (0xC0, 0xC1):
            p, h, w, nc = struct.unpack(">BHHB", seg[:6])
            comps = []
            for k in range(nc):
                cid, hv, tq = seg[6 + 3 * k:9 + 3 * k]
                comps.append({"id": cid, "h": hv >> 4, "v": hv & 15, "tq": tq})
            frame = (h, w, comps)
        elif m in (0xC2, 0xC3, 0xC5, 0xC6, 0xC7, 0xC9, 0xCA, 0xCB):
            raise ValueError("only baseline (sequential Huffman) JPEG is supported")
        elif m == 0xDD:
            restart = struct.unpack(">H", seg[:2])[0]
        elif m == 0xDA:
            ns = seg[0]
            for k in range(ns):
                cid, tt = seg[1 + 2 * k], seg[2 + 2 * k]
                for c in frame[2]:
                    if c["id"] == cid:
                        c["td"], c["ta"] = tt >> 4, tt & 15
            return _decode_scan(buf, pos + n, frame, qt, hdc, hac, restart)
        pos += n
    raise ValueError("JPEG without a scan")


def _decode_scan(buf, pos, frame, qt, hdc, hac, restart) -> np.ndarray:
    h, w, comps = frame
    hmax = max(c["h"] for c in comps)
    vmax = max(c["v"] for c in comps)
    mcux, mcuy = (w + 8 * hmax - 1) // (8 * hmax), (h + 8 * vmax - 1) // (8 * vmax)
    planes = [np.zeros((mcuy * c["v"] * 8, mcux * c["h"] * 8), dtype=np.float32) for c in comps]
    coefs = [np.zeros((mcuy * c["v"], mcux * c["h"], 64), dtype=np.int32) for c in comps]
    br = _Bits(buf, pos)
    pred = [0] * len(comps)
    count = 0
    for my in range(mcuy):
        for mx in range(mcux):
            if restart and count and count % restart == 0:
                br.reset()
                pred = [0] * len(comps)
            count += 1
            for ci, c in enumerate(comps):
                dc_t, ac_t = hdc[c["td"]], hac[c["ta"]]
                for by in range(c["v"]):
                    for bx in range(c["h"]):
                        blk = coefs[ci][my * c["v"] + by, mx * c["h"] + bx]
                        t = _huff(br, dc_t)
                        pred[ci] += _extend(br.get(t), t)
                        blk[0] = pred[ci]
                        k = 1
                        while k < 64:
                            rs = _huff(br, ac_t)
                            r, s = rs >> 4, rs & 15
                            if s == 0:
                                if r != 15:
                                    break
                                k += 16
                                continue
                            k += r
                            if k > 63:
                                break
                            blk[_ZZ[k]] = _extend(br.get(s), s)
                            k += 1
    for ci, c in enumerate(comps):
        q = qt[c["tq"]].astype(np.float32)
        blocks = coefs[ci].reshape(coefs[ci].shape[0], coefs[ci].shape[1], 8, 8).astype(np.float32) * q
        px = np.einsum("ki,yxkl,lj->yxij", _D, blocks, _D) + 128.0
        planes[ci] = px.transpose(0, 2, 1, 3).reshape(px.shape[0] * 8, px.shape[1] * 8)
    full = []
    for ci, c in enumerate(comps):
        p = planes[ci]
        ry, rx = vmax // c["v"], hmax // c["h"]
        if ry > 1 or rx > 1:
            p = np.repeat(np.repeat(p, ry, 0), rx, 1)
        full.append(p[:h, :w])
    if len(full) == 1:
        return np.clip(full[0] + 0.5, 0, 255).astype(np.uint8)[..., None]
    y, cb, cr = full[0], full[1] - 128.0, full[2] - 128.0
    rgb = np.stack([y + 1.402 * cr, y - 0.344136 * cb - 0.714136 * cr, y + 1.772 * cb], -1)
    return np.clip(rgb + 0.5, 0, 255).astype(np.uint8)


# ---- encoder ---------------------------------------------------------------------------------------------
def _scaled(q: np.ndarray, quality: int) -> np.ndarray:
    quality = max(1, min(100, int(quality)))
    s = 5000 // quality if quality < 50 else 200 - 2 * quality
    return np.clip((q * s + 50) // 100, 1, 255).astype(np.int32)


class _Writer:
    def __init__(self):
        self.out, self.acc, self.n = bytearray(), 0, 0

    def put(self, code: int, length: int):
        self.acc = (self.acc << length) | (code & ((1 << length) - 1))
        self.n += length
        while self.n >= 8:
            self.n -= 8
            b = (self.acc >> self.n) & 255
            self.out.append(b)
            if b == 0xFF:
                self.out.append(0)
        self.acc &= (1 << self.n) - 1

    def flush(self):
        if self.n:
            self.put((1 << (8 - self.n)) - 1, 8 - self.n)


def _category(v: int):
    a = -v if v < 0 else v
    t = a.bit_length()
    return t, (v if v >= 0 else v + (1 << t) - 1)


def encode_jpeg(a: np.ndarray, quality: int = 90) -> bytes:
    """``a`` is HxWx1 grey or HxWx3 RGB uint8."""
    if a.ndim == 2:
        a = a[..., None]
    h, w, c = a.shape
    f = a[..., :3].astype(np.float32) if c >= 3 else a[..., :1].astype(np.float32)
    if c >= 3:
        r, g, b = f[..., 0], f[..., 1], f[..., 2]
        planes = [0.299 * r + 0.587 * g + 0.114 * b,
                  -0.168736 * r - 0.331264 * g + 0.5 * b + 128.0,
                  0.5 * r - 0.418688 * g - 0.081312 * b + 128.0]
    else:
        planes = [f[..., 0]]
    ql, qc = _scaled(_Q_LUM, quality), _scaled(_Q_CHR, quality)
    H8, W8 = (h + 7) // 8 * 8, (w + 7) // 8 * 8
    coefs = []
    for i, p in enumerate(planes):
        p = np.pad(p, ((0, H8 - h), (0, W8 - w)), mode="edge") - 128.0
        blocks = p.reshape(H8 // 8, 8, W8 // 8, 8).transpose(0, 2, 1, 3)
        d = np.einsum("ik,yxkl,jl->yxij", _D, blocks, _D)
        q = (ql if i == 0 else qc).reshape(8, 8)
        coefs.append(np.rint(d / q).astype(np.int32).reshape(H8 // 8, W8 // 8, 64)[..., _ZZ])
    out = bytearray(b"\xff\xd8")
    out += b"\xff\xe0" + struct.pack(">H5sBBBHHBB", 16, b"JFIF\0", 1, 1, 0, 1, 1, 0, 0)
    for tid, q in ((0, ql), (1, qc))[:len(planes) if len(planes) == 1 else 2]:
        out += b"\xff\xdb" + struct.pack(">HB", 67, tid) + bytes(int(v) for v in q[_ZZ])
    nc = len(planes)
    out += b"\xff\xc0" + struct.pack(">HBHHB", 8 + 3 * nc, 8, h, w, nc)
    for i in range(nc):
        out += bytes([i + 1, 0x11, 0 if i == 0 else 1])
    tables = [(0x00, _DC_LUM), (0x10, _AC_LUM)] + ([(0x01, _DC_CHR), (0x11, _AC_CHR)] if nc > 1 else [])
    for tid, (bits, vals) in tables:
        out += b"\xff\xc4" + struct.pack(">HB", 19 + len(vals), tid) + bytes(bits) + bytes(vals)
    out += b"\xff\xda" + struct.pack(">HB", 6 + 2 * nc, nc)
    for i in range(nc):
        out += bytes([i + 1, 0x00 if i == 0 else 0x11])
    out += b"\x00\x3f\x00"
    dc = [_codes(*_DC_LUM), _codes(*_DC_CHR)]
    ac = [_codes(*_AC_LUM), _codes(*_AC_CHR)]
    wr = _Writer()
    pred = [0] * nc
    for by in range(H8 // 8):
        for bx in range(W8 // 8):
            for i in range(nc):
                t = 0 if i == 0 else 1
                blk = coefs[i][by, bx]
                diff = int(blk[0]) - pred[i]
                pred[i] = int(blk[0])
                cat, bits = _category(diff)
                wr.put(*dc[t][cat])
                if cat:
                    wr.put(bits, cat)
                nz = np.nonzero(blk[1:])[0]
                last = int(nz[-1]) + 1 if len(nz) else 0
                run = 0
                for k in range(1, last + 1):
                    v = int(blk[k])
                    if v == 0:
                        run += 1
                        continue
                    while run > 15:
                        wr.put(*ac[t][0xF0])
                        run -= 16
                    cat, bits = _category(v)
                    wr.put(*ac[t][(run << 4) | cat])
                    wr.put(bits, cat)
                    run = 0
                if last < 63:
                    wr.put(*ac[t][0x00])
    wr.flush()
    return bytes(out) + bytes(wr.out) + b"\xff\xd9"
