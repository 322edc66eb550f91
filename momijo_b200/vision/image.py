"""Image container of the vision package: packed HWC uint8 pixels in a torch tensor that may live
in host or device memory, plus the small metadata record the reference carries around
(legacy/src/momijo/vision/image.mojo:23-100 ``ImageMeta``, :102-470 ``Image``).

The reference stores a raw pointer with explicit strides; here the strides are the tensor's and
``ensure_packed_hwc_u8`` is a ``contiguous()`` call. Pixel accessors exist for API parity and for
tests; bulk work goes through the kernels in ``momijo_b200.vision.kernels``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Tuple

import numpy as np
import torch


class _Name(str):
    """An upper-case tag that compares as a string and, when called, gives the reference's spelling:
    ``cs.name == "GRAY"`` and ``cs.name() == "Gray"`` (legacy/src/momijo/vision/dtypes.mojo:142-148, 201-209)."""
    _ref = {"LINEAR": "Linear", "GRAY": "Gray", "YCBCR": "YCbCr", "UNKNOWN": "Unknown"}

    def __call__(self) -> str:
        return self._ref.get(str(self), str(self))


class ColorSpace:
    """Enumeration by name (legacy/src/momijo/vision/dtypes.mojo ``ColorSpace``)."""
    _names = ("SRGB", "LINEAR", "GRAY", "BGR", "RGB", "HSV", "YCBCR", "UNKNOWN")

    def __init__(self, name: str = "SRGB"):
        name = name.upper()
        if name not in self._names:
            raise ValueError(f"unknown colour space {name!r}")
        self.name = _Name(name)

    def copy(self) -> "ColorSpace":
        return ColorSpace(self.name)

    @staticmethod
    def from_name(name: str):
        """``(found, value)``: the reference's spellings and the upper-case tags; unknown names give
        ``(False, Unknown)`` (dtypes.mojo:211-218)."""
        up = name.upper()
        if up in ColorSpace._names:
            return True, ColorSpace(up)
        return False, ColorSpace("UNKNOWN")

    def __eq__(self, other):
        return isinstance(other, ColorSpace) and other.name == self.name

    def __hash__(self):
        return hash(self.name)

    def __repr__(self):
        return f"ColorSpace.{self.name}"


for _n in ColorSpace._names:
    setattr(ColorSpace, _n, staticmethod(lambda _n=_n: ColorSpace(_n)))
for _alias, _n in (("Linear", "LINEAR"), ("Gray", "GRAY"), ("YCbCr", "YCBCR"), ("Unknown", "UNKNOWN")):
    setattr(ColorSpace, _alias, staticmethod(lambda _n=_n: ColorSpace(_n)))


class Layout:
    _names = ("HWC", "CHW", "PLANAR")

    def __init__(self, name: str = "HWC"):
        name = name.upper()
        if name not in self._names:
            raise ValueError(f"unknown layout {name!r}")
        self.name = _Name(name)

    def copy(self) -> "Layout":
        return Layout(self.name)

    @staticmethod
    def from_name(name: str):
        """``(found, value)``; unknown names give ``(False, HWC)`` (dtypes.mojo:150-155)."""
        if name in Layout._names:
            return True, Layout(name)
        return False, Layout("HWC")

    def __eq__(self, other):
        return isinstance(other, Layout) and other.name == self.name

    def __hash__(self):
        return hash(self.name)

    def __repr__(self):
        return f"Layout.{self.name}"


Layout.HWC = staticmethod(lambda: Layout("HWC"))
Layout.CHW = staticmethod(lambda: Layout("CHW"))
Layout.PLANAR = staticmethod(lambda: Layout("PLANAR"))


@dataclass
class ImageMeta:
    _layout: Layout = None
    _colorspace: ColorSpace = None
    _premultiplied: bool = False

    def __post_init__(self):
        self._layout = self._layout or Layout.HWC()
        self._colorspace = self._colorspace or ColorSpace.SRGB()

    def copy(self):
        return replace(self)

    def layout(self):
        return self._layout

    def colorspace(self):
        return self._colorspace

    def is_premultiplied(self):
        return self._premultiplied

    alpha_premultiplied = is_premultiplied

    def with_colorspace(self, cs):
        return replace(self, _colorspace=cs)

    def with_layout(self, layout):
        return replace(self, _layout=layout)

    def with_premultiplied(self, v):
        return replace(self, _premultiplied=bool(v))

    def set_colorspace(self, cs):
        self._colorspace = cs

    def set_layout(self, layout):
        self._layout = layout

    def set_premultiplied(self, v):
        self._premultiplied = bool(v)

    def __str__(self):
        return f"ImageMeta(layout={self._layout.name}, cs={self._colorspace.name}, premul={self._premultiplied})"


def _as_hwc(t) -> torch.Tensor:
    if isinstance(t, Image):
        return t.data
    if isinstance(t, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(t))
    if not isinstance(t, torch.Tensor):
        t = torch.as_tensor(t)
    if t.dim() == 2:
        t = t.unsqueeze(-1)
    if t.dim() != 3:
        raise ValueError(f"an image is [H, W] or [H, W, C]; got shape {tuple(t.shape)}")
    return t


class Image:
    """HWC image; ``data`` is a torch tensor (uint8 for everything the transforms accept)."""

    def __init__(self, data, meta: ImageMeta = None):
        if isinstance(data, ImageMeta):  # reference argument order: Image(meta, tensor)
            data, meta = meta, data
        self.data = _as_hwc(data)
        self._meta = meta or ImageMeta()

    # ---- constructors ----
    @staticmethod
    def new_hwc_u8(h, w, c, value=0, cs: ColorSpace = None, layout: Layout = None, device=None):
        t = torch.full((max(int(h), 0), max(int(w), 0), max(int(c), 0)), int(value) & 255,
                       dtype=torch.uint8, device=device)
        return Image(t, ImageMeta(layout, cs))

    @staticmethod
    def from_numpy(a, cs: ColorSpace = None):
        return Image(torch.from_numpy(np.ascontiguousarray(a)), ImageMeta(None, cs))

    # ---- properties ----
    def tensor(self):
        return self.data

    def meta(self):
        return self._meta

    def height(self):
        return int(self.data.shape[0])

    def width(self):
        return int(self.data.shape[1])

    def channels(self):
        return int(self.data.shape[2])

    h = property(height)
    w = property(width)
    c = property(channels)

    @property
    def shape(self):
        return tuple(self.data.shape)

    @property
    def device(self):
        return self.data.device

    def dtype(self):
        return self.data.dtype

    def colorspace(self):
        return self._meta.colorspace()

    def layout(self):
        return self._meta.layout()

    def is_empty(self):
        return self.data.numel() == 0

    def is_hwc(self):
        return self._meta.layout() == Layout.HWC()

    def is_u8(self):
        return self.data.dtype == torch.uint8

    def is_contiguous_hwc_u8(self):
        return self.is_hwc() and self.is_u8() and self.data.is_contiguous()

    def ensure_packed_hwc_u8(self, force: bool = True):
        if self.is_contiguous_hwc_u8():
            return self
        t = self.data
        if t.dtype != torch.uint8:
            t = t.clamp(0, 255).to(torch.uint8)
        return Image(t.contiguous(), self._meta.copy())

    def clone(self):
        return Image(self.data.clone(), self._meta.copy())

    copy = clone

    def to(self, device):
        return Image(self.data.to(device), self._meta.copy())

    def cuda(self):
        return self.to("cuda")

    def cpu(self):
        return self.to("cpu")

    def numpy(self):
        return self.data.detach().cpu().numpy()

    def roi(self, y, x, h, w):
        """View of a rectangle clipped to the image (shares storage, like the reference's)."""
        y0, x0 = max(int(y), 0), max(int(x), 0)
        y1, x1 = min(int(y) + int(h), self.height()), min(int(x) + int(w), self.width())
        return Image(self.data[y0:max(y1, y0), x0:max(x1, x0)], self._meta.copy())

    def as_hwc_view(self, h: int = 0, w: int = 0, c: int = 0, s0: int = 0, s1: int = 0, s2: int = 0) -> "Image":
        """The reference returns a copy whatever the arguments (legacy/src/momijo/vision/image.mojo:262-263)."""
        return self.clone()

    def with_meta(self, meta):
        return Image(self.data, meta)

    def with_colorspace(self, cs):
        return Image(self.data, self._meta.with_colorspace(cs))

    # ---- pixel access ----
    def _inb(self, y, x, k):
        return 0 <= y < self.height() and 0 <= x < self.width() and 0 <= k < self.channels()

    def set_u8(self, y, x, k, v):
        if self._inb(y, x, k):
            self.data[y, x, k] = int(v) & 255

    def get_u8(self, y, x, k):
        return int(self.data[y, x, k]) if self._inb(y, x, k) else 0

    at_u8 = get_u8
    unsafe_set_u8 = set_u8
    unsafe_get_u8 = get_u8

    def set_rgb_u8(self, y, x, r, g, b):
        for k, v in enumerate((r, g, b)):
            self.set_u8(y, x, k, v)

    def get_rgb_u8(self, y, x) -> Tuple[int, int, int]:
        return self.get_u8(y, x, 0), self.get_u8(y, x, 1), self.get_u8(y, x, 2)

    # ---- alpha ----
    def premultiply_alpha(self):
        if self.channels() != 4 or self._meta.is_premultiplied():
            return self.clone()
        d = self.data.to(torch.int32)
        a = d[..., 3:4]
        rgb = (d[..., :3] * a + 127) // 255
        return Image(torch.cat([rgb, a], -1).to(torch.uint8), self._meta.with_premultiplied(True))

    def unpremultiply_alpha(self):
        if self.channels() != 4 or not self._meta.is_premultiplied():
            return self.clone()
        d = self.data.to(torch.int32)
        a = d[..., 3:4]
        rgb = torch.where(a > 0, (d[..., :3] * 255 + a // 2) // a.clamp(min=1), torch.zeros_like(d[..., :3]))
        return Image(torch.cat([rgb.clamp(0, 255), a], -1).to(torch.uint8), self._meta.with_premultiplied(False))

    def dump_table(self, max_rows: int = 0, max_cols: int = 0):
        a = self.numpy()
        rows = a.shape[0] if max_rows <= 0 else min(max_rows, a.shape[0])
        cols = a.shape[1] if max_cols <= 0 else min(max_cols, a.shape[1])
        for y in range(rows):
            print(" ".join("(" + ",".join(f"{int(v):3d}" for v in a[y, x]) + ")" for x in range(cols)))

    def __str__(self):
        return (f"Image(h={self.height()}, w={self.width()}, c={self.channels()}, dtype={self.data.dtype}, "
                f"device={self.data.device}, {self._meta})")

    __repr__ = __str__


def new_hwc_u8(h, w, c, value=0, cs=None, layout=None):
    return Image.new_hwc_u8(h, w, c, value, cs, layout)


def full_hwc_u8(h, w, c, value):
    return Image.new_hwc_u8(h, w, c, value)


def zeros_hwc_u8(h, w, c):
    return Image.new_hwc_u8(h, w, c, 0)


def make_zero_u8_hwc(h, w, c, cs=None):
    return Image.new_hwc_u8(h, w, c, 0, cs)


def make_u8_hwc(data, h: int, w: int, c: int, cs: ColorSpace = None) -> Image:
    """Image over an existing packed HWC uint8 buffer (tensor, bytes, bytearray or numpy array) without
    copying where possible; an invalid shape gives an empty image
    (legacy/src/momijo/vision/image.mojo:613-626)."""
    if h <= 0 or w <= 0 or c <= 0:
        return Image(torch.zeros(0, 0, 0, dtype=torch.uint8), ImageMeta(None, cs))
    from .tensor import tensor_from_u8_array_hwc
    t = data.reshape(h, w, c) if isinstance(data, torch.Tensor) else tensor_from_u8_array_hwc(data, h * w * c, h, w, c)
    return Image(t, ImageMeta(None, cs))


def validate_image(img: Image) -> bool:
    return isinstance(img, Image) and img.data.dim() == 3 and min(img.shape) > 0
