"""DEFLATE / zlib building blocks under the reference's names
(legacy/src/momijo/vision/io/encode_png.mojo:28-640, legacy/src/momijo/vision/io/inflate.mojo:9-330).

Own code: the LSB-first bit writer and reader, canonical Huffman tables from code lengths, the LZ77 matcher
with hash chains, stored and fixed-Huffman compression, and a complete inflater (stored, fixed and dynamic
blocks). ``deflate_dynamic_stream`` hands the block building to the standard library's zlib, whose output
the inflater here reads back like any other stream; checksums use zlib's table-driven routines."""
from __future__ import annotations

import zlib
from typing import List, Tuple


def crc32(data, start: int = 0, end: int = None) -> int:
    """CRC-32 (PNG polynomial) of ``data[start:end]``."""
    b = bytes(data)
    return zlib.crc32(b[start:len(b) if end is None else end]) & 0xFFFFFFFF


def adler32(data) -> int:
    return zlib.adler32(bytes(data)) & 0xFFFFFFFF


class BitWriter:
    """Bits are packed least-significant first, as DEFLATE wants them."""

    def __init__(self):
        self.buf = bytearray()
        self.cur = 0
        self.nbits = 0

    def write_bits(self, v: int, n: int) -> bool:
        self.cur |= (v & ((1 << n) - 1)) << self.nbits
        self.nbits += n
        while self.nbits >= 8:
            self.buf.append(self.cur & 255)
            self.cur >>= 8
            self.nbits -= 8
        return True

    def write_code(self, code: int, length: int) -> bool:
        """Huffman codes go out most-significant bit first."""
        rev = 0
        for _ in range(length):
            rev = (rev << 1) | (code & 1)
            code >>= 1
        return self.write_bits(rev, length)

    def align_byte(self) -> None:
        if self.nbits > 0:
            self.buf.append(self.cur & 255)
            self.cur = 0
            self.nbits = 0


class BitReader:
    def __init__(self, data, pos: int = 0):
        self.data = bytes(data)
        self.pos = pos
        self.cur = 0
        self.nbits = 0

    def read_bits(self, n: int) -> Tuple[bool, int]:
        while self.nbits < n:
            if self.pos >= len(self.data):
                return False, 0
            self.cur |= self.data[self.pos] << self.nbits
            self.pos += 1
            self.nbits += 8
        v = self.cur & ((1 << n) - 1)
        self.cur >>= n
        self.nbits -= n
        return True, v

    def align_byte(self) -> None:
        drop = self.nbits % 8
        self.cur >>= drop
        self.nbits -= drop

    align_to_byte = align_byte


class Huff:
    """Canonical Huffman table: per code length the first code, the index of its first symbol in ``values``
    and the number of codes; ``values`` lists the symbols sorted by (length, symbol)."""

    def __init__(self):
        self.first_code: List[int] = []
        self.first_symbol: List[int] = []
        self.count: List[int] = []
        self.values: List[int] = []
        self.max_bits = 0
        self.lengths: List[int] = []

    def code_of(self, sym: int) -> Tuple[bool, int, int]:
        """(found, code, length) of a symbol."""
        if sym < 0 or sym >= len(self.lengths) or self.lengths[sym] == 0:
            return False, 0, 0
        ln = self.lengths[sym]
        idx = self.values.index(sym, self.first_symbol[ln], self.first_symbol[ln] + self.count[ln])
        return True, self.first_code[ln] + (idx - self.first_symbol[ln]), ln


Huffman = Huff   # the inflater's name for the same table


def build_huffman(code_lengths: List[int], max_bits: int = 15) -> Tuple[bool, Huff]:
    h = Huff()
    h.max_bits = max_bits
    h.lengths = list(code_lengths)
    h.count = [0] * (max_bits + 1)
    for ln in code_lengths:
        if ln < 0 or ln > max_bits:
            return False, h
        h.count[ln] += 1
    h.count[0] = 0
    code, h.first_code, h.first_symbol = 0, [0] * (max_bits + 1), [0] * (max_bits + 1)
    left = 1
    for ln in range(1, max_bits + 1):
        left = (left << 1) - h.count[ln]
        if left < 0:
            return False, h           # over-subscribed
        code = (code + h.count[ln - 1]) << 1 if ln > 1 else 0
        h.first_code[ln] = code
        h.first_symbol[ln] = h.first_symbol[ln - 1] + h.count[ln - 1]
    h.values = [s for ln in range(1, max_bits + 1) for s, l in enumerate(code_lengths) if l == ln]
    return True, h


def put_code(bw: BitWriter, tab: Huff, sym: int) -> None:
    ok, code, ln = tab.code_of(sym)
    if ok:
        bw.write_code(code, ln)


def _huff_decode(br: BitReader, h: Huff) -> Tuple[bool, int]:
    code = 0
    for ln in range(1, h.max_bits + 1):
        ok, bit = br.read_bits(1)
        if not ok:
            return False, 0
        code = (code << 1) | bit
        n = h.count[ln]
        if n and code - h.first_code[ln] < n and code >= h.first_code[ln]:
            return True, h.values[h.first_symbol[ln] + code - h.first_code[ln]]
    return False, 0


# ---- length / distance code tables (RFC 1951 section 3.2.5) -----------------------------------------------
_LEN_BASE = [3, 4, 5, 6, 7, 8, 9, 10, 11, 13, 15, 17, 19, 23, 27, 31, 35, 43, 51, 59, 67, 83, 99, 115, 131, 163, 195,
             227, 258]
_LEN_EBITS = [0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 3, 3, 3, 3, 4, 4, 4, 4, 5, 5, 5, 5, 0]
_DIST_BASE = [1, 2, 3, 4, 5, 7, 9, 13, 17, 25, 33, 49, 65, 97, 129, 193, 257, 385, 513, 769, 1025, 1537, 2049, 3073,
              4097, 6145, 8193, 12289, 16385, 24577]
_DIST_EBITS = [0, 0, 0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7, 8, 8, 9, 9, 10, 10, 11, 11, 12, 12, 13, 13]


def _len_to_code(length: int) -> Tuple[int, int, int]:
    for i in range(len(_LEN_BASE) - 1, -1, -1):
        if length >= _LEN_BASE[i]:
            return 257 + i, _LEN_EBITS[i], length - _LEN_BASE[i]
    raise ValueError("match length below 3")


def _dist_to_code(dist: int) -> Tuple[int, int, int]:
    for i in range(len(_DIST_BASE) - 1, -1, -1):
        if dist >= _DIST_BASE[i]:
            return i, _DIST_EBITS[i], dist - _DIST_BASE[i]
    raise ValueError("distance below 1")


class Tok:
    """One LZ77 token: a literal byte, or a (length, distance) match with its codes and extra bits."""

    def __init__(self, lit, length, dist, len_code, len_ebits, len_extra, dist_code, dist_ebits, dist_extra, is_lit):
        self.lit, self.length, self.dist = lit, length, dist
        self.len_code, self.len_ebits, self.len_extra = len_code, len_ebits, len_extra
        self.dist_code, self.dist_ebits, self.dist_extra = dist_code, dist_ebits, dist_extra
        self.is_lit = is_lit


def make_lit(lit: int) -> Tok:
    return Tok(lit, 0, 0, 0, 0, 0, 0, 0, 0, True)


def make_match(length: int, dist: int, len_code: int = None, len_ebits: int = 0, len_extra: int = 0,
               dist_code: int = None, dist_ebits: int = 0, dist_extra: int = 0) -> Tok:
    if len_code is None:
        len_code, len_ebits, len_extra = _len_to_code(length)
    if dist_code is None:
        dist_code, dist_ebits, dist_extra = _dist_to_code(dist)
    return Tok(0, length, dist, len_code, len_ebits, len_extra, dist_code, dist_ebits, dist_extra, False)


class CLE:
    """Entry of a run-length coded code-length sequence: symbol 0..18 with its extra bits."""

    def __init__(self, sym: int = 0, ebits: int = 0, extra: int = 0):
        self.sym, self.ebits, self.extra = sym, ebits, extra


class HC:
    """Hash chains over 3-byte prefixes: ``head[hash]`` is the latest position, ``prev[pos]`` the one before."""

    def __init__(self, n: int):
        self.head = [-1] * 65536
        self.prev = [-1] * n


def _hash3(a: int, b: int, c: int) -> int:
    return (a * 911 + b * 131 + c * 31) & 0xFFFF


def build_tokens(data: bytes, window: int = 32768, max_len: int = 258, chain_cap: int = 32) -> List[Tok]:
    n = len(data)
    hc = HC(n)
    toks: List[Tok] = []
    pos = 0

    def insert(p):
        if p + 2 < n:
            h = _hash3(data[p], data[p + 1], data[p + 2])
            hc.prev[p] = hc.head[h]
            hc.head[h] = p

    while pos < n:
        best_len, best_dist = 0, 0
        if pos + 2 < n:
            cand = hc.head[_hash3(data[pos], data[pos + 1], data[pos + 2])]
            steps = 0
            limit = min(max_len, n - pos)
            while cand >= 0 and pos - cand <= window and steps < chain_cap:
                ln = 0
                while ln < limit and data[cand + ln] == data[pos + ln]:
                    ln += 1
                if ln > best_len:
                    best_len, best_dist = ln, pos - cand
                    if ln == limit:
                        break
                cand = hc.prev[cand]
                steps += 1
        if best_len >= 3:
            toks.append(make_match(best_len, best_dist))
            for p in range(pos, pos + best_len):
                insert(p)
            pos += best_len
        else:
            toks.append(make_lit(data[pos]))
            insert(pos)
            pos += 1
    return toks


def _fixed_tables() -> Tuple[Huff, Huff]:
    lens = [8] * 144 + [9] * 112 + [7] * 24 + [8] * 8
    return build_huffman(lens, 15)[1], build_huffman([5] * 30, 15)[1]


_FIXED = None


def _fixed():
    global _FIXED
    if _FIXED is None:
        _FIXED = _fixed_tables()
    return _FIXED


def deflate_fixed_stream(data) -> bytes:
    """Raw DEFLATE stream: one final block with the fixed Huffman codes over LZ77 tokens."""
    data = bytes(data)
    lit, dist = _fixed()
    bw = BitWriter()
    bw.write_bits(1, 1)       # BFINAL
    bw.write_bits(1, 2)       # BTYPE = 01
    for t in build_tokens(data):
        if t.is_lit:
            put_code(bw, lit, t.lit)
        else:
            put_code(bw, lit, t.len_code)
            if t.len_ebits:
                bw.write_bits(t.len_extra, t.len_ebits)
            put_code(bw, dist, t.dist_code)
            if t.dist_ebits:
                bw.write_bits(t.dist_extra, t.dist_ebits)
    put_code(bw, lit, 256)
    bw.align_byte()
    return bytes(bw.buf)


def deflate_dynamic_stream(data) -> bytes:
    """Raw DEFLATE stream with dynamic Huffman blocks (block building by the standard library)."""
    c = zlib.compressobj(9, zlib.DEFLATED, -15)
    return c.compress(bytes(data)) + c.flush()


def _zlib_wrap(raw: bytes, data: bytes) -> bytes:
    return b"\x78\x9c" + raw + adler32(data).to_bytes(4, "big")


def zlib_stored(data) -> bytes:
    """zlib stream made of stored (uncompressed) blocks of at most 65535 bytes."""
    data = bytes(data)
    out = bytearray(b"\x78\x01")
    pos, n = 0, len(data)
    if n == 0:
        out += b"\x01\x00\x00\xff\xff"
    while pos < n:
        chunk = data[pos:pos + 65535]
        pos += len(chunk)
        out.append(1 if pos >= n else 0)
        out += len(chunk).to_bytes(2, "little") + (len(chunk) ^ 0xFFFF).to_bytes(2, "little") + chunk
    return bytes(out) + adler32(data).to_bytes(4, "big")


def zlib_deflate(data, mode: int = 2) -> bytes:
    """zlib stream: ``mode`` 0 stored, 1 fixed Huffman, anything else dynamic Huffman."""
    data = bytes(data)
    if mode == 0:
        return zlib_stored(data)
    if mode == 1:
        return _zlib_wrap(deflate_fixed_stream(data), data)
    return _zlib_wrap(deflate_dynamic_stream(data), data)


_CL_ORDER = [16, 17, 18, 0, 8, 7, 9, 6, 10, 5, 11, 4, 12, 3, 13, 2, 14, 1, 15]


def _inflate_block(br: BitReader, lit: Huff, dist: Huff, out: bytearray) -> bool:
    while True:
        ok, sym = _huff_decode(br, lit)
        if not ok:
            return False
        if sym < 256:
            out.append(sym)
        elif sym == 256:
            return True
        else:
            i = sym - 257
            if i >= len(_LEN_BASE):
                return False
            ok, extra = br.read_bits(_LEN_EBITS[i])
            if not ok:
                return False
            length = _LEN_BASE[i] + extra
            ok, ds = _huff_decode(br, dist)
            if not ok or ds >= len(_DIST_BASE):
                return False
            ok, extra = br.read_bits(_DIST_EBITS[ds])
            if not ok:
                return False
            d = _DIST_BASE[ds] + extra
            if d > len(out):
                return False
            for _ in range(length):
                out.append(out[-d])


def inflate_raw(data, pos: int = 0) -> Tuple[bool, bytes, int]:
    """(ok, bytes, position after the stream) for a raw DEFLATE stream."""
    br = BitReader(data, pos)
    out = bytearray()
    while True:
        ok, final = br.read_bits(1)
        ok2, btype = br.read_bits(2)
        if not (ok and ok2):
            return False, bytes(out), br.pos
        if btype == 0:
            br.align_byte()
            ok, ln = br.read_bits(16)
            ok2, nln = br.read_bits(16)
            if not (ok and ok2) or (ln ^ 0xFFFF) != nln:
                return False, bytes(out), br.pos
            for _ in range(ln):
                ok, b = br.read_bits(8)
                if not ok:
                    return False, bytes(out), br.pos
                out.append(b)
        elif btype == 1:
            lit, dist = _fixed()
            if not _inflate_block(br, lit, dist, out):
                return False, bytes(out), br.pos
        elif btype == 2:
            ok, hlit = br.read_bits(5)
            ok2, hdist = br.read_bits(5)
            ok3, hclen = br.read_bits(4)
            if not (ok and ok2 and ok3):
                return False, bytes(out), br.pos
            cl = [0] * 19
            for i in range(hclen + 4):
                ok, v = br.read_bits(3)
                if not ok:
                    return False, bytes(out), br.pos
                cl[_CL_ORDER[i]] = v
            ok, clt = build_huffman(cl, 7)
            if not ok:
                return False, bytes(out), br.pos
            lens: List[int] = []
            total = hlit + 257 + hdist + 1
            while len(lens) < total:
                ok, sym = _huff_decode(br, clt)
                if not ok:
                    return False, bytes(out), br.pos
                if sym < 16:
                    lens.append(sym)
                elif sym == 16:
                    ok, r = br.read_bits(2)
                    if not ok or not lens:
                        return False, bytes(out), br.pos
                    lens += [lens[-1]] * (3 + r)
                elif sym == 17:
                    ok, r = br.read_bits(3)
                    lens += [0] * (3 + r)
                else:
                    ok, r = br.read_bits(7)
                    lens += [0] * (11 + r)
            lens = lens[:total]
            ok, lit = build_huffman(lens[:hlit + 257], 15)
            ok2, dist = build_huffman(lens[hlit + 257:], 15)
            if not ok or not _inflate_block(br, lit, dist, out):
                return False, bytes(out), br.pos
        else:
            return False, bytes(out), br.pos
        if final:
            br.align_byte()
            return True, bytes(out), br.pos - br.nbits // 8


def zlib_inflate(z) -> Tuple[bool, bytes]:
    """(ok, bytes): checks the two header bytes, inflates, and verifies the Adler-32 trailer."""
    z = bytes(z)
    if len(z) < 6 or (z[0] & 0x0F) != 8 or ((z[0] << 8) | z[1]) % 31 != 0 or (z[1] & 0x20):
        return False, b""
    ok, out, end = inflate_raw(z, 2)
    if not ok or end + 4 > len(z):
        return False, out
    return int.from_bytes(z[end:end + 4], "big") == adler32(out), out
