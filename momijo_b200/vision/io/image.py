"""File-level image I/O with format detection by signature and by extension
(legacy/src/momijo/vision/io/image.mojo:1-179, registry.mojo, image_read.mojo, image_write.mojo).
Colour images are RGB in memory unless ``bgr=True`` is asked for."""
from __future__ import annotations

import os
from typing import Callable, Dict, Tuple

import numpy as np
import torch

from ..image import ColorSpace, Image, ImageMeta
from . import jpeg as _jpeg
from . import png as _png
from . import ppm as _ppm

_DECODERS: Dict[str, Callable[[bytes], np.ndarray]] = {}
_ENCODERS: Dict[str, Callable[..., bytes]] = {}


def register_codec(name: str, decode: Callable = None, encode: Callable = None) -> None:
    if decode is not None:
        _DECODERS[name] = decode
    if encode is not None:
        _ENCODERS[name] = encode


register_codec("png", _png.decode_png, _png.encode_png)
register_codec("jpeg", _jpeg.decode_jpeg, _jpeg.encode_jpeg)
register_codec("ppm", _ppm.decode_ppm, _ppm.encode_ppm)


def sniff_format(buf: bytes) -> str:
    if buf[:8] == b"\x89PNG\r\n\x1a\n":
        return "png"
    if buf[:2] == b"\xff\xd8":
        return "jpeg"
    if buf[:2] in (b"P2", b"P3", b"P5", b"P6"):
        return "ppm"
    return ""


def format_from_path(path: str) -> str:
    ext = os.path.splitext(path)[1].lower()
    return {".png": "png", ".jpg": "jpeg", ".jpeg": "jpeg", ".ppm": "ppm", ".pgm": "ppm", ".pnm": "ppm"}.get(ext, "")


def decode_image(buf: bytes, bgr: bool = False) -> Image:
    fmt = sniff_format(buf)
    if not fmt:
        raise ValueError("unrecognised image format")
    a = _DECODERS[fmt](buf)
    if bgr and a.shape[2] >= 3:
        a = np.ascontiguousarray(a[..., [2, 1, 0] + list(range(3, a.shape[2]))])
    cs = ColorSpace("GRAY") if a.shape[2] == 1 else ColorSpace("BGR" if bgr else "RGB")
    return Image(torch.from_numpy(np.ascontiguousarray(a)), ImageMeta(None, cs))


def read_image_any(path: str, bgr: bool = False) -> Tuple[bool, Image]:
    """``(ok, image)``; a 1x1 black image comes back with ``ok == False`` (image.mojo's contract)."""
    try:
        with open(path, "rb") as f:
            return True, decode_image(f.read(), bgr)
    except (OSError, ValueError, KeyError, IndexError):
        return False, Image.new_hwc_u8(1, 1, 1, 0)


def read_image(path: str, bgr: bool = False) -> Image:
    with open(path, "rb") as f:
        return decode_image(f.read(), bgr)


imread = read_image


def encode_image(img: Image, fmt: str, **kw) -> bytes:
    a = img.ensure_packed_hwc_u8().numpy()
    if img.colorspace() == ColorSpace("BGR") and a.shape[2] >= 3:
        a = np.ascontiguousarray(a[..., [2, 1, 0] + list(range(3, a.shape[2]))])
    if fmt == "jpeg" and a.shape[2] == 4:
        a = a[..., :3]
    if fmt == "ppm" and a.shape[2] == 2:
        a = a[..., :1]
    return _ENCODERS[fmt](a, **kw)


def write_image_any(path: str, img: Image, **kw) -> bool:
    fmt = format_from_path(path) or "png"
    try:
        data = encode_image(img, fmt, **kw)
        with open(path, "wb") as f:
            f.write(data)
        return True
    except (OSError, ValueError, KeyError):
        return False


def write_image(path: str, img: Image, interlace: int = 0, compress: int = 2, filter_mode: int = -1,
                palette_mode: int = 0, max_colors: int = 256, bit_depth_out: int = 8, **kw) -> bool:
    """Format by file extension. The PNG tuning arguments of the reference (legacy/src/momijo/vision/io/
    image_write.mojo:8-11) are accepted in its order; this encoder writes non-interlaced 8-bit true-colour / grey
    images with per-row filters and takes no tuning, so they are not used."""
    return write_image_any(path, img, **kw)


imwrite = write_image


def read_png(path: str) -> Image:
    with open(path, "rb") as f:
        return Image(torch.from_numpy(_png.decode_png(f.read())))


def write_png(path: str, img: Image, interlace: int = 0, compress: int = 2, filter_mode: int = -1,
              palette_mode: int = 0, max_colors: int = 256, bit_depth_out: int = 8) -> bool:
    """PNG file; the tuning arguments are accepted as in ``write_image``."""
    return write_image_any(path if path.lower().endswith(".png") else path + ".png", img)


def read_jpeg(path: str) -> Image:
    with open(path, "rb") as f:
        return Image(torch.from_numpy(_jpeg.decode_jpeg(f.read())))


def write_jpeg(path: str, img: Image, quality: int = 90) -> bool:
    return write_image_any(path, img, quality=quality)


def read_ppm(path: str) -> Image:
    with open(path, "rb") as f:
        return Image(torch.from_numpy(_ppm.decode_ppm(f.read())))


def write_ppm(path: str, img: Image) -> bool:
    return write_image_any(path, img)


# ---- readers with a synthetic fallback (legacy/src/momijo/vision/io/registry.mojo:18-190,
# legacy/src/momijo/vision/io/image.mojo:26-46, legacy/src/momijo/vision/io/jpeg.mojo:60-121, 246-270).
# They return (ok, uint8 HWC tensor); when nothing decodes, ``ok`` is False and the tensor is the
# reference's test pattern (y*7 + x*11 + ch*29) mod 256, so downstream code still has pixels to work on.
def make_dummy_u8_hwc_tensor(h: int = 32, w: int = 32, c: int = 3, default: int = 32) -> torch.Tensor:
    h = h if h > 0 else default
    w = w if w > 0 else default
    c = c if c in (1, 3) else 3
    y = torch.arange(h)[:, None, None]
    x = torch.arange(w)[None, :, None]
    ch = torch.arange(c)[None, None, :]
    return ((y * 7 + x * 11 + ch * 29) % 256).to(torch.uint8)


def unsafe_char_from_code(code: int) -> str:
    return chr(code) if 0 <= code < 0x110000 else "?"


def _try_decode(path: str, fmts) -> Tuple[bool, torch.Tensor]:
    try:
        with open(path, "rb") as f:
            buf = f.read()
    except OSError:
        return False, None
    for fmt in fmts:
        try:
            return True, torch.from_numpy(np.ascontiguousarray(_DECODERS[fmt](buf)))
        except Exception:       # a decoder rejecting foreign bytes is the expected case here
            continue
    return False, None


def _order_for(path: str):
    p = path.lower()
    if p.endswith((".jpg", ".jpeg", ".jpe")):
        return ("jpeg", "png")
    if p.endswith(".png"):
        return ("png", "jpeg")
    if p.endswith((".ppm", ".pgm")):
        return ("ppm", "jpeg", "png")
    return ("jpeg", "png")


def read_image_auto(path: str) -> Tuple[bool, torch.Tensor]:
    """Decoder chosen by extension, the other formats tried next; a 32 x 32 x 3 pattern on failure."""
    ok, t = _try_decode(path, _order_for(path))
    return (True, t) if ok else (False, make_dummy_u8_hwc_tensor(32, 32, 3))


def read_image_auto_with_fallback(path: str, fallback_h: int = 64, fallback_w: int = 64, fallback_c: int = 3):
    ok, t = _try_decode(path, _order_for(path))
    return (True, t) if ok else (False, make_dummy_u8_hwc_tensor(fallback_h, fallback_w, fallback_c, 64))


def read_image_with_fallback(path: str, fallback_h: int = 64, fallback_w: int = 64, fallback_c: int = 3):
    ok, t = _try_decode(path, ("png", "jpeg", "ppm"))
    return (True, t) if ok else (False, make_dummy_u8_hwc_tensor(fallback_h, fallback_w, fallback_c, 64))


def has_jpeg_codec() -> bool:
    return "jpeg" in _DECODERS


def read_jpeg_with_fallback(path: str, fallback_h: int = 64, fallback_w: int = 64, fallback_c: int = 3):
    ok, t = _try_decode(path, ("jpeg",))
    return (True, t) if ok else (False, make_dummy_u8_hwc_tensor(fallback_h, fallback_w, fallback_c, 64))


def read_jpeg_image(path: str) -> Image:
    """Decoded image, or the 64 x 64 x 3 pattern as an Image when the file cannot be decoded."""
    ok, t = read_jpeg_with_fallback(path)
    cs = ColorSpace("GRAY") if t.shape[2] == 1 else ColorSpace("RGB")
    return Image(t, ImageMeta(None, cs))


def write_jpeg_image(path: str, img: Image, quality: int = 90) -> bool:
    return write_jpeg(path, img, quality)
