"""Baseline-JPEG building blocks under the reference's names: marker and segment parsing
(legacy/src/momijo/vision/io/jpeg_decoder.mojo:19-205), the 8 x 8 DCT pair (jpeg_dct.mojo:164, idct.mojo:12-140),
quantisation and zig-zag (jpeg_quantize.mojo:18-100), BT.601 colour conversion (color_ycbcr.mojo:8-100), the
Annex K tables (tables.mojo, jpeg_huffman_encode.mojo:85-155), entropy coding of one block
(jpeg_huffman_encode.mojo:158-230, huffman.mojo:12-75, jpeg_scan.mojo:37-110), the MSB-first bit reader and
writer with byte stuffing (bitreader.mojo, bitwriter.mojo) and the header writers (jpeg_writer.mojo:22-245).

Pointers of the reference became Python sequences: functions that filled an output pointer return the result
instead. The whole-file codec that uses the same tables is ``momijo_b200.vision.io.jpeg``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

from .jpeg import _AC_CHR, _AC_LUM, _D, _DC_CHR, _DC_LUM, _Q_CHR, _Q_LUM, _ZZ


# ---- markers and segments ---------------------------------------------------------------------------------
def MARK_SOI() -> int: return 0xFFD8     # noqa: E704
def MARK_EOI() -> int: return 0xFFD9     # noqa: E704
def MARK_APP0() -> int: return 0xFFE0    # noqa: E704
def MARK_APP1() -> int: return 0xFFE1    # noqa: E704
def MARK_DQT() -> int: return 0xFFDB     # noqa: E704
def MARK_SOF0() -> int: return 0xFFC0    # noqa: E704
def MARK_DHT() -> int: return 0xFFC4     # noqa: E704
def MARK_SOS() -> int: return 0xFFDA     # noqa: E704
def MARK_TEM() -> int: return 0xFF01     # noqa: E704
def MARK_RST0() -> int: return 0xFFD0    # noqa: E704


def read_be_u16(buf, off: int = 0) -> int:
    return (buf[off] << 8) | buf[off + 1]


def is_jpeg(buf, off: int = 0) -> bool:
    return len(buf) >= off + 2 and buf[off] == 0xFF and buf[off + 1] == 0xD8


def is_rst(marker: int) -> bool:
    return MARK_RST0() <= marker <= MARK_RST0() + 7


def has_length_field(marker: int) -> bool:
    """SOI, EOI, TEM and RST0..7 stand alone; every other marker is followed by a 2-byte length."""
    return not (marker in (MARK_SOI(), MARK_EOI(), MARK_TEM()) or is_rst(marker))


@dataclass
class JpegSegment:
    marker: int
    length: int          # value of the length field (counts its own two bytes)
    data: bytes          # payload (length - 2 bytes); the reference keeps a pointer
    offset: int = 0      # where the payload starts in the file


@dataclass
class ParseSegResult:
    ok: bool
    seg: JpegSegment


def parse_segment(buf, off: int = 0, end: int = None) -> ParseSegResult:
    """Segment whose 0xFF byte sits at ``off``; ``ok`` is False when it is truncated or its length is bad."""
    b = bytes(buf)
    end = len(b) if end is None else end
    if off + 4 > end:
        return ParseSegResult(False, JpegSegment(0, 0, b"", off))
    marker, length = read_be_u16(b, off), read_be_u16(b, off + 2)
    if length < 2 or off + 2 + length > end:
        return ParseSegResult(False, JpegSegment(marker, length, b"", off + 4))
    return ParseSegResult(True, JpegSegment(marker, length, b[off + 4:off + 2 + length], off + 4))


def parse_sof0_dims(payload, payload_len: int = None) -> Tuple[bool, int, int, int]:
    """(ok, width, height, components) from a SOF0 payload; only 8-bit precision is accepted."""
    n = len(payload) if payload_len is None else payload_len
    if n < 6:
        return False, 0, 0, 0
    precision, height, width, nf = payload[0], read_be_u16(payload, 1), read_be_u16(payload, 3), payload[5]
    if n < 6 + 3 * nf or precision != 8 or width <= 0 or height <= 0:
        return False, 0, 0, 0
    return True, width, height, nf


_NAMES = {0xFFD8: "SOI", 0xFFD9: "EOI", 0xFFE0: "APP0", 0xFFE1: "APP1", 0xFFDB: "DQT", 0xFFC0: "SOF0", 0xFFC2: "SOF2",
          0xFFC4: "DHT", 0xFFDA: "SOS", 0xFFDD: "DRI", 0xFFFE: "COM"}


def inspect_jpeg_structure(buf, length: int = None, emit=print) -> List[Tuple[str, int, int]]:
    """Walk the marker segments up to the first scan; prints one line per segment and returns
    (name, file offset, length field) triples."""
    b = bytes(buf)
    n = len(b) if length is None else min(length, len(b))
    out: List[Tuple[str, int, int]] = []
    if not is_jpeg(b):
        emit("not a JPEG stream")
        return out
    pos = 0
    while pos + 2 <= n:
        if b[pos] != 0xFF:
            pos += 1
            continue
        marker = read_be_u16(b, pos)
        name = _NAMES.get(marker, f"0x{marker:04X}")
        if not has_length_field(marker):
            out.append((name, pos, 0))
            emit(f"{name} @ {pos}")
            pos += 2
            if marker == MARK_EOI():
                break
            continue
        r = parse_segment(b, pos, n)
        if not r.ok:
            emit(f"{name} @ {pos}: truncated")
            break
        extra = ""
        if marker == MARK_SOF0():
            ok, w, h, nf = parse_sof0_dims(r.seg.data)
            extra = f" {w}x{h}x{nf}" if ok else " (unsupported frame)"
        out.append((name, pos, r.seg.length))
        emit(f"{name} @ {pos} len {r.seg.length}{extra}")
        pos += 2 + r.seg.length
        if marker == MARK_SOS():
            break
    return out


# ---- DCT, quantisation, zig-zag ---------------------------------------------------------------------------
def dct_8x8(src, stride: int = 8, off: int = 0) -> List[int]:
    """Forward DCT of the 8 x 8 window at ``off`` of a single-channel uint8 buffer with row pitch ``stride``
    (level shift by 128 first); 64 rounded coefficients in natural (row-major) order."""
    a = np.asarray(src, dtype=np.float64).reshape(-1)
    blk = np.stack([a[off + y * stride: off + y * stride + 8] for y in range(8)]) - 128.0
    return np.rint(_D @ blk @ _D.T).astype(np.int64).reshape(-1).tolist()


def descale(x: int, n: int) -> int:
    return (x + (1 << (n - 1))) >> n


def idct_8x8(data: List[int]) -> List[int]:
    """Inverse DCT in place: 64 coefficients (natural order) become 64 samples centred on zero (add 128 and
    clamp to get pixels). Returns ``data``."""
    blk = np.asarray(data, dtype=np.float64).reshape(8, 8)
    out = np.rint(_D.T @ blk @ _D).astype(np.int64).reshape(-1).tolist()
    data[:] = out
    return data


def _qdiv(val: int, q: int) -> int:
    q = max(int(q), 1)
    return (val + q // 2) // q if val >= 0 else -((-val + q // 2) // q)


def quantize_block(dct: Sequence[int], quant: Sequence[int]) -> List[int]:
    """Round-half-away division of each coefficient by its quantiser (both in natural order)."""
    return [_qdiv(int(dct[i]), int(quant[i])) for i in range(64)]


def zigzag_copy(src: Sequence[int]) -> List[int]:
    """natural order -> zig-zag order: out[z] = src[ZIGZAG[z]]."""
    return [src[int(_ZZ[z])] for z in range(64)]


def inv_zigzag_copy(src: Sequence[int]) -> List[int]:
    out = [0] * 64
    for z in range(64):
        out[int(_ZZ[z])] = src[z]
    return out


# ---- colour ---------------------------------------------------------------------------------------------
def rgb_to_ycbcr(src, w: int, h: int):
    """Packed RGB (HWC uint8) -> three planes (Y, Cb, Cr) of w*h bytes each, BT.601 full range in 8-bit fixed
    point: Y = (77 R + 150 G + 29 B + 128) >> 8, Cb = ((-43 R - 85 G + 128 B + 128) >> 8) + 128,
    Cr = ((128 R - 107 G - 21 B + 128) >> 8) + 128, clamped."""
    a = np.frombuffer(bytes(src), dtype=np.uint8)[: w * h * 3].reshape(-1, 3).astype(np.int64)
    r, g, b = a[:, 0], a[:, 1], a[:, 2]
    y = (77 * r + 150 * g + 29 * b + 128) >> 8
    cb = ((-43 * r - 85 * g + 128 * b + 128) >> 8) + 128
    cr = ((128 * r - 107 * g - 21 * b + 128) >> 8) + 128
    cl = lambda v: np.clip(v, 0, 255).astype(np.uint8).tobytes()
    return cl(y), cl(cb), cl(cr)


def merge_ycbcr_to_rgb(y, cb, cr, width: int, height: int) -> bytes:
    """Planes -> packed RGB: R = Y + 91881 Cr' / 65536, G = Y - (22554 Cb' + 46802 Cr') / 65536,
    B = Y + 116130 Cb' / 65536 with Cb' = Cb - 128, Cr' = Cr - 128; the divisions truncate toward zero."""
    n = width * height
    Y = np.frombuffer(bytes(y), dtype=np.uint8)[:n].astype(np.int64)
    Cb = np.frombuffer(bytes(cb), dtype=np.uint8)[:n].astype(np.int64) - 128
    Cr = np.frombuffer(bytes(cr), dtype=np.uint8)[:n].astype(np.int64) - 128
    tdiv = lambda v: np.sign(v) * (np.abs(v) // 65536)
    r = Y + tdiv(91881 * Cr)
    g = Y - tdiv(22554 * Cb + 46802 * Cr)
    b = Y + tdiv(116130 * Cb)
    return np.clip(np.stack([r, g, b], -1), 0, 255).astype(np.uint8).tobytes()


# ---- Annex K tables -----------------------------------------------------------------------------------------
def std_luma_qt() -> List[int]: return [int(v) for v in _Q_LUM]            # noqa: E704
def std_chroma_qt() -> List[int]: return [int(v) for v in _Q_CHR]          # noqa: E704
def std_dc_lengths_luma() -> List[int]: return list(_DC_LUM[0])            # noqa: E704
def std_dc_symbols_luma() -> List[int]: return list(_DC_LUM[1])            # noqa: E704
def std_dc_lengths_chroma() -> List[int]: return list(_DC_CHR[0])          # noqa: E704
def std_dc_symbols_chroma() -> List[int]: return list(_DC_CHR[1])          # noqa: E704
def std_ac_lengths_luma() -> List[int]: return list(_AC_LUM[0])            # noqa: E704
def std_ac_symbols_luma() -> List[int]: return list(_AC_LUM[1])            # noqa: E704
def std_ac_lengths_chroma() -> List[int]: return list(_AC_CHR[0])          # noqa: E704
def std_ac_symbols_chroma() -> List[int]: return list(_AC_CHR[1])          # noqa: E704


std_dc_lengths, std_dc_symbols = std_dc_lengths_luma, std_dc_symbols_luma
std_ac_lengths, std_ac_symbols = std_ac_lengths_luma, std_ac_symbols_luma
bits_dc_luma, bits_dc_chroma = std_dc_lengths_luma, std_dc_lengths_chroma
bits_ac_luma, bits_ac_chroma = std_ac_lengths_luma, std_ac_lengths_chroma
vals_ac_luma, vals_ac_chroma = std_ac_symbols_luma, std_ac_symbols_chroma


def vals_dc_common() -> List[int]:
    return list(range(12))


# ---- Huffman coding ---------------------------------------------------------------------------------------------
@dataclass
class HuffCode:
    code: int = 0     # MSB-first code bits
    size: int = 0     # code length in bits


def build_canonical_codes(bits: Sequence[int], vals: Sequence[int]) -> List[HuffCode]:
    """Canonical codes in ``vals`` order from the 16 per-length counts."""
    sizes = [i + 1 for i in range(16) for _ in range(int(bits[i]))]
    codes: List[HuffCode] = []
    code = 0
    for k, si in enumerate(sizes):
        if k > 0:
            code <<= si - sizes[k - 1]
        codes.append(HuffCode(code, si))
        code += 1
    return codes


def expand_ac(vals: Sequence[int], codes: Sequence[HuffCode]) -> List[HuffCode]:
    """256-entry table indexed by the run/size symbol."""
    table = [HuffCode(0, 0) for _ in range(256)]
    for j, sym in enumerate(vals):
        table[int(sym)] = codes[j]
    return table


def expand_dc(codes: Sequence[HuffCode]) -> List[HuffCode]:
    """12-entry table indexed by the DC category."""
    return [codes[k] for k in range(12)]


def build_default_codebooks():
    """(DC luma, DC chroma, AC luma, AC chroma) lookup tables of the Annex K codes."""
    dcl = expand_dc(build_canonical_codes(bits_dc_luma(), vals_dc_common()))
    dcc = expand_dc(build_canonical_codes(bits_dc_chroma(), vals_dc_common()))
    acl = expand_ac(vals_ac_luma(), build_canonical_codes(bits_ac_luma(), vals_ac_luma()))
    acc = expand_ac(vals_ac_chroma(), build_canonical_codes(bits_ac_chroma(), vals_ac_chroma()))
    return dcl, dcc, acl, acc


def dc_mag_bits(v: int) -> Tuple[int, int]:
    """(category, additional bits): negatives are stored as the one's complement of their magnitude."""
    if v == 0:
        return 0, 0
    a = abs(v)
    n = a.bit_length()
    return n, (a if v >= 0 else (~a) & ((1 << n) - 1))


class BitWriter:
    """MSB-first bit packing with JPEG byte stuffing (a zero byte follows every 0xFF data byte)."""

    def __init__(self, cap: int = None):
        self.buf = bytearray()
        self.cap = cap
        self.bit_acc = 0
        self.bit_count = 0
        self.ok = True

    @property
    def pos(self) -> int:
        return len(self.buf)

    def _put_byte(self, b: int) -> bool:
        if self.cap is not None and len(self.buf) >= self.cap:
            self.ok = False
            return False
        self.buf.append(b & 255)
        return True

    def write_u8(self, b: int) -> bool:
        """Raw byte (markers, header fields): no stuffing; call on a byte boundary."""
        return self._put_byte(b)

    def write_bits(self, bits: int, nbits: int) -> bool:
        if nbits <= 0 or nbits > 16:
            self.ok = False
            return False
        self.bit_acc = (self.bit_acc << nbits) | (bits & ((1 << nbits) - 1))
        self.bit_count += nbits
        while self.bit_count >= 8:
            self.bit_count -= 8
            outb = (self.bit_acc >> self.bit_count) & 0xFF
            if not self._put_byte(outb) or (outb == 0xFF and not self._put_byte(0)):
                return False
        self.bit_acc &= (1 << self.bit_count) - 1
        return True

    def byte_align(self) -> bool:
        """Pad with zero bits to the next byte boundary, as the reference does."""
        return True if self.bit_count == 0 else self.write_bits(0, 8 - self.bit_count)

    def tell(self) -> int:
        return self.pos

    def good(self) -> bool:
        return self.ok


class BitReader:
    """MSB-first reader over entropy-coded data: removes stuffed zero bytes and stops at a marker."""

    def __init__(self, data, length: int = None):
        self.reset(data, length)

    def reset(self, data, length: int = None):
        self.data = bytes(data)
        self.length = len(self.data) if length is None else min(length, len(self.data))
        self.pos = 0
        self.bit_buf = 0
        self.bit_count = 0
        self.eof_flag = False

    def is_eof(self) -> bool:
        return self.eof_flag

    def bytes_consumed(self) -> int:
        return self.pos

    def remaining_bytes(self) -> int:
        return max(self.length - self.pos, 0)

    def _fill(self, need: int):
        while self.bit_count < need and not self.eof_flag:
            if self.pos >= self.length:
                self.eof_flag = True
                break
            b = self.data[self.pos]
            if b == 0xFF:
                if self.pos + 1 < self.length and self.data[self.pos + 1] == 0:
                    self.pos += 2
                else:
                    self.eof_flag = True          # a marker: leave it for the caller
                    break
            else:
                self.pos += 1
            self.bit_buf = (self.bit_buf << 8) | b
            self.bit_count += 8

    def read_bits(self, n: int) -> int:
        """Next ``n`` bits (0 bits are supplied past the end, with ``is_eof()`` set)."""
        if n <= 0:
            return 0
        self._fill(n)
        if self.bit_count < n:
            self.bit_buf <<= n - self.bit_count
            self.bit_count = n
        self.bit_count -= n
        v = (self.bit_buf >> self.bit_count) & ((1 << n) - 1)
        self.bit_buf &= (1 << self.bit_count) - 1
        return v

    # ---- the rest of the reference's reader (legacy/src/momijo/vision/io/bitreader.mojo:112-185) ------------------
    def read_bit(self) -> int:
        return self.read_bits(1)

    def peek_bits(self, n: int) -> int:
        """Next ``n`` bits without consuming them; 0 when fewer are left."""
        if n <= 0:
            return 0
        self._fill(min(n, 24))
        if self.bit_count < n:
            return 0
        return (self.bit_buf >> (self.bit_count - n)) & ((1 << n) - 1)

    def skip_bits(self, n: int) -> None:
        if n <= 0:
            return
        self._fill(n)
        if self.bit_count < n:
            self.bit_buf, self.bit_count, self.eof_flag = 0, 0, True
            return
        self.bit_count -= n
        self.bit_buf &= (1 << self.bit_count) - 1

    def align_byte(self) -> None:
        rem = self.bit_count % 8
        if rem:
            self.read_bits(rem)

    def read_data_byte(self):
        """``(ok, byte)`` straight from the stream after aligning: a stuffed ``FF 00`` gives ``FF``; a marker or the end
        gives ``(False, 0)`` and sets the end flag."""
        self.align_byte()
        if self.bit_count >= 8:                      # whole bytes already buffered come first
            return True, self.read_bits(8)
        if self.eof_flag or self.pos >= self.length:
            self.eof_flag = True
            return False, 0
        b = self.data[self.pos]
        self.pos += 1
        if b == 0xFF:
            if self.pos < self.length and self.data[self.pos] == 0:
                self.pos += 1
                return True, 0xFF
            self.eof_flag = True
            return False, 0
        return True, b


class HuffmanTable:
    """Decoder-side table: codes ordered by length then value, with sizes and symbols alongside."""

    def __init__(self):
        self.codes: List[int] = []
        self.sizes: List[int] = []
        self.symbols: List[int] = []
        self._lut = {}

    def build(self, counts: Sequence[int], symbols: Sequence[int]):
        code, idx = 0, 0
        for si in range(1, 17):
            for _ in range(int(counts[si - 1])):
                self.codes.append(code)
                self.sizes.append(si)
                self.symbols.append(int(symbols[idx]))
                self._lut[(si, code)] = int(symbols[idx])
                code += 1
                idx += 1
            code <<= 1
        return self

    def decode(self, br: BitReader) -> int:
        acc = 0
        for ln in range(1, 17):
            acc = (acc << 1) | br.read_bits(1)
            sym = self._lut.get((ln, acc))
            if sym is not None:
                return sym
        return -1


def receive_extend(br: BitReader, s: int) -> int:
    """``s`` additional bits as a signed value (values below 2^(s-1) are negative)."""
    if s == 0:
        return 0
    val = br.read_bits(s)
    return val - ((1 << s) - 1) if val < (1 << (s - 1)) else val


def encode_block(bw: BitWriter, zz: Sequence[int], is_luma: bool, prev_dc: int, dcL, dcC, acL, acC) -> int:
    """Entropy-code one quantised block given in zig-zag order; returns the block's DC value (the next
    block's predictor)."""
    dc_t, ac_t = (dcL, acL) if is_luma else (dcC, acC)
    nbits, add = dc_mag_bits(int(zz[0]) - prev_dc)
    h = dc_t[min(max(nbits, 0), 11)]
    bw.write_bits(h.code, h.size)
    if nbits > 0:
        bw.write_bits(add, nbits)
    run = 0
    for k in range(1, 64):
        v = int(zz[k])
        if v == 0:
            run += 1
            continue
        while run >= 16:
            bw.write_bits(ac_t[0xF0].code, ac_t[0xF0].size)
            run -= 16
        n, add = dc_mag_bits(v)
        h = ac_t[(run << 4) | n]
        bw.write_bits(h.code, h.size)
        bw.write_bits(add, n)
        run = 0
    if run > 0:
        bw.write_bits(ac_t[0x00].code, ac_t[0x00].size)
    return int(zz[0])


def decode_block(br: BitReader, dc_table: HuffmanTable, ac_table: HuffmanTable, quant: Sequence[int], prev_dc: int,
                 dst: List[int]) -> int:
    """Decode, dequantise and inverse-transform one block into ``dst`` (64 samples centred on zero, natural
    order). Returns the block's DC value, or -1 when the bit stream is invalid."""
    coef = [0] * 64
    t = dc_table.decode(br)
    if t < 0:
        return -1
    dc = prev_dc + receive_extend(br, t)
    coef[0] = dc * int(quant[0])
    k = 1
    while k < 64:
        rs = ac_table.decode(br)
        if rs < 0:
            return -1
        if rs == 0:
            break
        if rs == 0xF0:
            k += 16
            continue
        k += rs >> 4
        if k > 63:
            return -1
        n = int(_ZZ[k])
        coef[n] = receive_extend(br, rs & 15) * int(quant[n])
        k += 1
    dst[:] = idct_8x8(coef)
    return dc


# ---- header writers -----------------------------------------------------------------------------------------
def write_u16_be(bw: BitWriter, v: int) -> bool:
    return bw.write_u8((v >> 8) & 255) and bw.write_u8(v & 255)


def _marker(bw: BitWriter, m: int) -> bool:
    return bw.write_u8(0xFF) and bw.write_u8(m & 255)


def write_soi(bw: BitWriter) -> bool:
    return _marker(bw, 0xD8)


def write_eoi(bw: BitWriter) -> bool:
    return _marker(bw, 0xD9)


def write_app0_jfif(bw: BitWriter, xdpi: int = 72, ydpi: int = 72) -> bool:
    ok = _marker(bw, 0xE0) and write_u16_be(bw, 16)
    for b in b"JFIF\x00\x01\x01\x01":
        ok = ok and bw.write_u8(b)
    return ok and write_u16_be(bw, xdpi) and write_u16_be(bw, ydpi) and bw.write_u8(0) and bw.write_u8(0)


def write_dqt(bw: BitWriter, table_id: int, table: Sequence[int]) -> bool:
    """One 8-bit quantisation table given in natural order (written in zig-zag order)."""
    ok = _marker(bw, 0xDB) and write_u16_be(bw, 67) and bw.write_u8(table_id & 15)
    for z in range(64):
        ok = ok and bw.write_u8(int(table[int(_ZZ[z])]))
    return ok


def _sof0(bw: BitWriter, width: int, height: int, comps) -> bool:
    ok = _marker(bw, 0xC0) and write_u16_be(bw, 8 + 3 * len(comps)) and bw.write_u8(8)
    ok = ok and write_u16_be(bw, height) and write_u16_be(bw, width) and bw.write_u8(len(comps))
    for cid, samp, tq in comps:
        ok = ok and bw.write_u8(cid) and bw.write_u8(samp) and bw.write_u8(tq)
    return ok


def write_sof0(bw: BitWriter, width: int, height: int) -> bool:
    """Grey frame: one component, 1x1 sampling, table 0."""
    return _sof0(bw, width, height, [(1, 0x11, 0)])


def write_sof0_color(bw: BitWriter, width: int, height: int) -> bool:
    """Y, Cb, Cr at 1x1 sampling (4:4:4); luma uses table 0, chroma table 1."""
    return _sof0(bw, width, height, [(1, 0x11, 0), (2, 0x11, 1), (3, 0x11, 1)])


def _dht(bw: BitWriter, tc: int, th: int, bits, vals) -> bool:
    ok = _marker(bw, 0xC4) and write_u16_be(bw, 2 + 1 + 16 + len(vals)) and bw.write_u8((tc << 4) | th)
    for b in bits:
        ok = ok and bw.write_u8(int(b))
    for v in vals:
        ok = ok and bw.write_u8(int(v))
    return ok


def write_dht_std(bw: BitWriter) -> bool:
    """The four Annex K tables: DC/AC for luma (id 0) and chroma (id 1)."""
    return (_dht(bw, 0, 0, bits_dc_luma(), vals_dc_common()) and _dht(bw, 1, 0, bits_ac_luma(), vals_ac_luma())
            and _dht(bw, 0, 1, bits_dc_chroma(), vals_dc_common()) and _dht(bw, 1, 1, bits_ac_chroma(), vals_ac_chroma()))


def _sos(bw: BitWriter, comps) -> bool:
    ok = _marker(bw, 0xDA) and write_u16_be(bw, 6 + 2 * len(comps)) and bw.write_u8(len(comps))
    for cid, tables in comps:
        ok = ok and bw.write_u8(cid) and bw.write_u8(tables)
    return ok and bw.write_u8(0) and bw.write_u8(63) and bw.write_u8(0)


def write_sos_gray(bw: BitWriter) -> bool:
    return _sos(bw, [(1, 0x00)])


def write_sos_color(bw: BitWriter) -> bool:
    return _sos(bw, [(1, 0x00), (2, 0x11), (3, 0x11)])
