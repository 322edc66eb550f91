"""Element types, layouts and colour spaces by name (legacy/src/momijo/vision/dtypes.mojo:22-229).

``DType`` numbers its seven members like the reference (UInt8 0, UInt16 1, Int32 2, Float16 3, Float32 4,
Int64 5, Float64 6) and maps each to the torch dtype that backs it here. ``Layout`` and ``ColorSpace`` are the
classes of ``momijo_b200.vision.image``; the functions below translate between them and the reference's names
(``"Linear"``, ``"Gray"``, ``"YCbCr"``, ...). The ``*_from_name`` functions return ``(found, value)`` with the
reference's fallback value when the name is unknown."""
from __future__ import annotations

import torch

from .image import ColorSpace, Layout

_NAMES = ("UInt8", "UInt16", "Int32", "Float16", "Float32", "Int64", "Float64")
_NBYTES = (1, 2, 4, 2, 4, 8, 8)
_TORCH = (torch.uint8, torch.uint16, torch.int32, torch.float16, torch.float32, torch.int64, torch.float64)


class DType:
    def __init__(self, id: int):
        self.id = int(id)

    def copy(self) -> "DType":
        return DType(self.id)

    def __eq__(self, other):
        return isinstance(other, DType) and other.id == self.id

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(("vision.DType", self.id))

    def name(self) -> str:
        return _NAMES[self.id] if 0 <= self.id < len(_NAMES) else "Unknown"

    def nbytes(self) -> int:
        return _NBYTES[self.id] if 0 <= self.id < len(_NBYTES) else 1

    def is_integer(self) -> bool:
        return self.id in (0, 1, 2, 5)

    def is_float(self) -> bool:
        return self.id in (3, 4, 6)

    def to_torch(self) -> torch.dtype:
        return _TORCH[self.id] if 0 <= self.id < len(_TORCH) else torch.uint8

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        return DType(_TORCH.index(dt)) if dt in _TORCH else DType(0)

    @staticmethod
    def from_name(name: str):
        return (True, DType(_NAMES.index(name))) if name in _NAMES else (False, DType(0))

    def __str__(self):
        return f"DType(id={self.id}, name={self.name()}, nbytes={self.nbytes()})"

    __repr__ = __str__


for _i, _n in enumerate(_NAMES):
    setattr(DType, _n, staticmethod(lambda _i=_i: DType(_i)))


def dtype_bytes(dt: DType) -> int:
    return dt.nbytes()


def dtype_name(dt: DType) -> str:
    return dt.name()


def dtype_from_name(name: str):
    return DType.from_name(name)


def dtype_is_integer(dt: DType) -> bool:
    return dt.is_integer()


def dtype_is_float(dt: DType) -> bool:
    return dt.is_float()


def layout_name(l: Layout) -> str:
    return l.name if l.name in ("HWC", "CHW", "PLANAR") else "Unknown"


def layout_from_name(name: str):
    if name in ("HWC", "CHW", "PLANAR"):
        return True, Layout(name)
    return False, Layout("HWC")


_CS_TO_REF = {"SRGB": "SRGB", "LINEAR": "Linear", "GRAY": "Gray", "YCBCR": "YCbCr", "UNKNOWN": "Unknown"}
_REF_TO_CS = {v: k for k, v in _CS_TO_REF.items()}


def colorspace_name(cs: ColorSpace) -> str:
    """The reference's spelling; colour spaces it does not have (BGR, RGB, HSV) keep their own name."""
    return _CS_TO_REF.get(cs.name, cs.name)


def colorspace_from_name(name: str):
    if name in _REF_TO_CS:
        return True, ColorSpace(_REF_TO_CS[name])
    return False, ColorSpace("UNKNOWN")
