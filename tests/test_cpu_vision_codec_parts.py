"""Byte-level codec parts, memory helpers and augmentations of the vision package (CPU)."""
import os
import random
import zlib

import numpy as np
import torch

from momijo_b200 import vision as V
from momijo_b200.vision import memory as M
from momijo_b200.vision.io import deflate as D, file_io as F, jpeg_parts as J, png as P
from momijo_b200.vision.io.jpeg import decode_jpeg


def test_deflate_and_inflate_agree_with_zlib():
    random.seed(1)
    cases = [b"", b"a", b"hello hello hello world" * 20, os.urandom(3000),
             bytes(random.choice(b"abc") for _ in range(2000)), bytes(70000)]
    for c in cases:
        for mode in (0, 1, 2):
            z = D.zlib_deflate(c, mode)
            assert zlib.decompress(z) == c
            ok, out = D.zlib_inflate(z)
            assert ok and out == c
        ok, out = D.zlib_inflate(zlib.compress(c, 9))
        assert ok and out == c
        assert zlib.decompress(D.deflate_fixed_stream(c), -15) == c
    assert D.crc32(b"abcdef", 1, 4) == zlib.crc32(b"bcd") and D.adler32(b"abc") == zlib.adler32(b"abc")
    assert not D.zlib_inflate(b"\x00" * 8)[0]
    ok, h = D.build_huffman([2, 1, 3, 3])
    assert ok and h.code_of(1) == (True, 0, 1) and h.code_of(0) == (True, 2, 2)
    assert not D.build_huffman([1, 1, 1])[0]          # over-subscribed


def test_png_byte_api_round_trip():
    a = np.random.RandomState(0).randint(0, 256, (5, 7, 3), dtype=np.uint8)
    for comp in (0, 1, 2):
        ok, b = P.png_from_hwc_u8(7, 5, 3, a.tobytes(), compress=comp)
        assert ok
        ok2, w, h, c, px = P.decode_png_bytes(b)
        assert ok2 and (w, h, c) == (7, 5, 3) and px == a.tobytes()
    ok, hdr = P.read_png_header_only(b)
    assert ok and (hdr.width, hdr.height, hdr.bit_depth, hdr.color_type) == (7, 5, 8, 2)
    assert P.parse_chunk(b, 8).type_str == "IHDR" and P.is_png_magic(b) and not P.decode_png_bytes(b"junk")[0]
    assert P.decode_png_bytes_u16(b)[4][:2] == [int(a[0, 0, 0]) * 257, int(a[0, 0, 1]) * 257]
    assert not P.png_from_hwc_u8(7, 5, 3, a.tobytes()[:-1])[0]
    scan = b"".join(b"\x00" + a[y].tobytes() for y in range(5))
    assert P.png_unfilter(7, 5, 3, scan) == (True, a.tobytes())


def test_jpeg_assembled_from_parts_decodes():
    yy, xx = np.mgrid[0:16, 0:24]
    img = (128 + 60 * np.sin(xx / 5.0) + 40 * np.cos(yy / 3.0)).clip(0, 255).astype(np.uint8)
    dcL, dcC, acL, acC = J.build_default_codebooks()
    bw = J.BitWriter()
    assert J.write_soi(bw) and J.write_app0_jfif(bw) and J.write_dqt(bw, 0, J.std_luma_qt())
    assert J.write_sof0(bw, 24, 16) and J.write_dht_std(bw) and J.write_sos_gray(bw)
    prev, flat = 0, img.reshape(-1)
    for by in range(2):
        for bx in range(3):
            q = J.quantize_block(J.dct_8x8(flat, 24, by * 8 * 24 + bx * 8), J.std_luma_qt())
            prev = J.encode_block(bw, J.zigzag_copy(q), True, prev, dcL, dcC, acL, acC)
    bw.byte_align()
    J.write_eoi(bw)
    data = bytes(bw.buf)
    out = decode_jpeg(data)
    assert out.shape == (16, 24, 1) and np.abs(out[..., 0].astype(int) - img.astype(int)).mean() < 3.0
    names = [n for n, _, _ in J.inspect_jpeg_structure(data, emit=lambda s: None)]
    assert names[:4] == ["SOI", "APP0", "DQT", "SOF0"] and names[-1] == "SOS"
    off = data.index(b"\xff\xda")
    seg = J.parse_segment(data, off)
    br = J.BitReader(data[off + 2 + seg.seg.length:])
    dct = J.HuffmanTable().build(J.std_dc_lengths_luma(), J.std_dc_symbols_luma())
    act = J.HuffmanTable().build(J.std_ac_lengths_luma(), J.std_ac_symbols_luma())
    dst = [0] * 64
    assert J.decode_block(br, dct, act, J.std_luma_qt(), 0, dst) >= 0
    assert np.abs(np.array(dst).reshape(8, 8) + 128 - img[:8, :8].astype(int)).mean() < 3.0
    assert J.inv_zigzag_copy(J.zigzag_copy(list(range(64)))) == list(range(64))
    assert J.dc_mag_bits(-5) == (3, 2) and J.dc_mag_bits(0) == (0, 0)
    assert J.parse_sof0_dims(bytes([8, 0, 16, 0, 24, 1, 1, 0x11, 0])) == (True, 24, 16, 1)
    assert not J.has_length_field(0xFFD3) and J.has_length_field(0xFFE0)
    y, cb, cr = J.rgb_to_ycbcr(bytes([255, 0, 0, 10, 10, 10]), 2, 1)
    assert list(y) == [77, 10] and list(cb)[1] == 128
    rgb = J.merge_ycbcr_to_rgb(y, cb, cr, 2, 1)
    assert abs(rgb[0] - 255) <= 2 and rgb[1] <= 3 and list(rgb[3:]) == [10, 10, 10]


def test_memfs_memory_and_fallback_readers(tmp_path):
    fs = F.MemFileStore()
    assert F.memfs_write_replace(fs, "x", b"abc")[:2] == (True, 3)
    assert F.memfs_append_ptr(fs, "x", b"defg", 2)[1] == 5 and F.memfs_try_read(fs, "x")[2] == b"abcde"
    assert F.memfs_list_all(fs)[3] == ["x"] and F.memfs_remove_path(fs, "x")[0] and not F.memfs_has_path(fs, "x")[0]
    b = M.BufferU8(16, True)
    b.write_from(bytes(range(8)), 8, 4)
    assert M.as_i32_view(b, 4)[1].item() == 0x03020100 and M.hexdump_head(b, 16, 6) == "00 00 00 00 00 01"
    assert M.memcmp_u8(b.slice(4, 4), bytes([0, 1, 2, 9]), 4) == -6 and M.byte_to_hex(171) == "AB"
    b.copy_range(4, 6, 6)
    assert b.data().tolist()[6:12] == [0, 1, 2, 3, 4, 5]
    img = V.Image(torch.randint(0, 256, (16, 16, 3), dtype=torch.uint8))
    V.write_png(str(tmp_path / "a.png"), img)
    ok, t = V.io.read_image_auto(str(tmp_path / "a.png"))
    assert ok and torch.equal(t, img.data)
    os.rename(tmp_path / "a.png", tmp_path / "c.jpg")       # wrong extension: the other decoder is tried
    assert V.io.read_image_auto(str(tmp_path / "c.jpg"))[0]
    ok, t = V.io.read_image_auto_with_fallback(str(tmp_path / "none.png"), 0, 5, 2)
    assert not ok and t.shape == (64, 5, 3) and int(t[1, 2, 1]) == (7 + 22 + 29) % 256


def test_augmentations_and_dtypes():
    torch.manual_seed(0)
    x = torch.randint(0, 256, (6, 8, 3), dtype=torch.uint8)
    assert torch.equal(V.ColorJitter(1, 1, 1, 0)(x), x)
    dark = V.ColorJitter(0.5, 1, 1, 0)(x)
    assert torch.equal(dark, (x.float() * 0.5 + 0.5).clamp(0, 255).to(torch.uint8))
    grey = V.ColorJitter(1, 1, 0.0, 0)(x)
    assert torch.equal(grey[..., 0], grey[..., 1]) and torch.equal(grey[..., 0], x.max(-1).values)
    flip = V.RandomHorizontalFlip(1.0)
    assert torch.equal(flip(x), x.flip(1)) and torch.equal(V.RandomHorizontalFlip(0.0)(x), x)
    assert torch.equal(V.RandomRotation(0.0)(x), x) and V.RandomRotation(30.0)(x).shape == x.shape
    r180 = V.transforms.random_ops._rotate_nearest_hwc_u8(x, 180.0)
    assert torch.equal(r180, x.flip(0).flip(1))
    assert V.RandomResizedCrop(4, 4)(x).shape == (4, 4, 3) and V.RandomResizedCrop(12, 12)(x).shape == (12, 12, 3)
    a, b = V.RandomResizedCrop(4, 4, seed=5), V.RandomResizedCrop(4, 4, seed=5)
    assert torch.equal(a(x), b(x))
    assert V.ToTensor()(x).shape == (3, 6, 8) and float(V.ToTensor()(x).max()) <= 1.0
    assert V.DType.Float32().nbytes() == 4 and V.dtype_from_name("Int64")[1].to_torch() == torch.int64
    assert V.layout_from_name("PLANAR")[0] and not V.layout_from_name("zzz")[0]
    assert V.colorspace_name(V.ColorSpace("YCBCR")) == "YCbCr" and not V.supports_windows()
    img = V.Image(x)
    assert V.run_single_op(V.OpKind.ResizeNearest, img, 3, 4, V.KernelRegistry(V.BackendKind.CPUSIMD)).shape == (3, 4, 3)
    assert V.run_single_op(99, img).shape == (6, 8, 3)
    assert V.backend.cpu.rgb_to_gray_u8_hwc(x).shape == (6, 8, 1)
    assert V.tensor_from_raw_chw(bytes(range(24)), 24, 3, 2, 4, V.DType.UInt8())[1, 0].tolist() == [8, 9, 10, 11]
