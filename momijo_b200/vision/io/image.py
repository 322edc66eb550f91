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


def write_image(path: str, img: Image, **kw) -> bool:
    return write_image_any(path, img, **kw)


imwrite = write_image


def read_png(path: str) -> Image:
    with open(path, "rb") as f:
        return Image(torch.from_numpy(_png.decode_png(f.read())))


def write_png(path: str, img: Image) -> bool:
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
