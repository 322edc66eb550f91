"""The vision package's own small tensor type is a strided raw pointer in the reference
(legacy/src/momijo/vision/tensor.mojo:35); here it is a torch tensor, and this module keeps the
helper names that code written against the reference imports."""
from __future__ import annotations

import torch

class Tensor(torch.Tensor):
    """An image buffer read through the reference's accessors (legacy/src/momijo/vision/tensor.mojo:28-290): height /
    width / channels (``shape0..2``), element strides, byte-level loads and stores, packed copies and region copies.
    It is a ``torch.Tensor`` subclass, so every function of this package takes it as it takes a plain tensor; wrap
    one with ``Tensor.wrap(t)``."""

    @staticmethod
    def wrap(t: torch.Tensor) -> "Tensor":
        return t.as_subclass(Tensor)

    def _dim(self, k: int) -> int:
        return int(self.shape[k]) if self.dim() > k else 0

    def height(self) -> int: return self._dim(0)
    def width(self) -> int: return self._dim(1)
    def channels(self) -> int: return self._dim(2)
    shape0, shape1, shape2 = height, width, channels

    def _stride(self, k: int) -> int:
        return int(self.stride(k)) if self.dim() > k else 0

    def stride0(self) -> int: return self._stride(0)
    def stride1(self) -> int: return self._stride(1)
    def stride2(self) -> int: return self._stride(2)

    def is_empty(self) -> bool:
        return self.numel() == 0

    def is_contiguous_hwc_u8(self) -> bool:
        return (self.dtype == torch.uint8 and self.dim() == 3
                and (self.stride2(), self.stride1(), self.stride0()) == (1, self.shape2(), self.shape1() * self.shape2()))

    def clone_deep(self) -> "Tensor":
        """Same bytes, same strides, own storage."""
        out = torch.empty_strided(tuple(self.shape), self.stride(), dtype=self.dtype, device=self.device)
        out.copy_(self)
        return Tensor.wrap(out)

    clone_bytes = clone_deep

    def copy_to_packed_hwc(self) -> "Tensor":
        return Tensor.wrap(self.contiguous().clone()) if self.numel() else Tensor.wrap(torch.empty(0, dtype=self.dtype))

    def ptr_u8(self) -> torch.Tensor:
        """The bytes of a dense buffer as a flat uint8 view (stands in for the raw pointer)."""
        return self.as_subclass(torch.Tensor).contiguous().view(-1).view(torch.uint8) if not self.is_contiguous() \
            else self.as_subclass(torch.Tensor).view(-1).view(torch.uint8)

    def store_u8_at(self, idx: int, v: int) -> None:
        self.ptr_u8()[idx] = int(v) & 0xFF

    def load_u8_at(self, idx: int) -> int:
        return int(self.ptr_u8()[idx])

    def copy_roi(self, y: int, x: int, h: int, w: int) -> "Tensor":
        """Packed copy of the ``h x w`` window at ``(y, x)``: the origin is clamped to 0, the size to what is left of
        the image, and an empty window gives an empty tensor (tensor.mojo:222-278)."""
        y, x = max(y, 0), max(x, 0)
        h, w = min(h, self.height() - y), min(w, self.width() - x)
        if h <= 0 or w <= 0:
            return Tensor.wrap(torch.empty(0, dtype=self.dtype))
        return Tensor.wrap(self.as_subclass(torch.Tensor)[y:y + h, x:x + w].contiguous().clone())


def packed_hwc_strides(h: int, w: int, c: int):
    return (w * c, c, 1)


def packed_chw_strides(c: int, h: int, w: int):
    return (h * w, w, 1)


# ---- constructors and raw-buffer adapters (legacy/src/momijo/vision/tensor.mojo:334-545 and
# legacy/src/momijo/vision/adapters/arrow.mojo:25-80). "Raw" means any object with the buffer protocol
# (bytes, bytearray, memoryview, numpy array) or a uint8 torch tensor; views share memory with it where
# torch allows, and invalid sizes give an empty tensor like the reference.
def _dt(dtype):
    from .dtypes import DType
    if dtype is None:
        return torch.uint8
    return dtype.to_torch() if isinstance(dtype, DType) else dtype


def dtype_bytes(dt) -> int:
    from .dtypes import DType
    return dt.nbytes() if isinstance(dt, DType) else torch.empty(0, dtype=dt).element_size()


def empty_1d(length: int, dtype=None) -> torch.Tensor:
    return torch.zeros(max(int(length), 0), dtype=_dt(dtype))


def empty_hwc(h: int, w: int, c: int, dtype=None) -> torch.Tensor:
    if h <= 0 or w <= 0 or c <= 0:
        return torch.zeros(0, dtype=_dt(dtype))
    return torch.zeros(h, w, c, dtype=_dt(dtype))


def _as_u8(raw) -> torch.Tensor:
    if isinstance(raw, torch.Tensor):
        return raw.reshape(-1).view(torch.uint8) if raw.dtype != torch.uint8 else raw.reshape(-1)
    if isinstance(raw, bytes):
        raw = bytearray(raw)          # torch wants a writable buffer
    return torch.frombuffer(raw, dtype=torch.uint8) if len(raw) else torch.zeros(0, dtype=torch.uint8)


def tensor_from_raw_strided(ptr, nbytes: int, d0: int, d1: int, d2: int, s0: int, s1: int, s2: int, dt=None):
    """[d0, d1, d2] view with element strides (s0, s1, s2) over a raw buffer."""
    if min(d0, d1, d2, s0, s1, s2, nbytes) <= 0:
        return torch.zeros(0, dtype=_dt(dt))
    flat = _as_u8(ptr)[:nbytes]
    td = _dt(dt)
    flat = flat[: flat.numel() // dtype_bytes(td) * dtype_bytes(td)].view(td)
    need = (d0 - 1) * s0 + (d1 - 1) * s1 + (d2 - 1) * s2 + 1
    if flat.numel() < need:
        return torch.zeros(0, dtype=td)
    return torch.as_strided(flat, (d0, d1, d2), (s0, s1, s2))


def unsafe_view_from_raw_u8(ptr, nbytes: int, h: int, w: int, c: int, s0: int, s1: int, s2: int, dt=None):
    return tensor_from_raw_strided(ptr, nbytes, h, w, c, s0, s1, s2, dt)


def tensor_from_u8_array_hwc(data, nbytes: int, h: int, w: int, c: int):
    if h <= 0 or w <= 0 or c <= 0 or nbytes < h * w * c:
        return torch.zeros(0, dtype=torch.uint8)
    return _as_u8(data)[: h * w * c].reshape(h, w, c)


def array_from_tensor_u8_hwc(t: torch.Tensor):
    """The tensor's bytes as a flat uint8 view (the reference hands back the data pointer)."""
    return t.contiguous().reshape(-1).view(torch.uint8)


def tensor_from_raw_chw(ptr, nbytes: int, c: int, h: int, w: int, dt=None):
    td = _dt(dt)
    if c <= 0 or h <= 0 or w <= 0 or nbytes < c * h * w * dtype_bytes(td):
        return torch.zeros(0, dtype=td)
    return _as_u8(ptr)[: c * h * w * dtype_bytes(td)].view(td).reshape(c, h, w)


def to_tensor_chw(src, h: int, w: int, c: int, scale: float = 1.0 / 255.0) -> torch.Tensor:
    """HWC uint8 (tensor or raw buffer) -> float32 CHW scaled by ``scale``."""
    from .transforms.random_ops import ToTensor
    return ToTensor(scale, True)(_as_u8(src) if not isinstance(src, torch.Tensor) else src, h, w, c)


def to_tensor_hwc(src, h: int, w: int, c: int, scale: float = 1.0 / 255.0) -> torch.Tensor:
    from .transforms.random_ops import ToTensor
    return ToTensor(scale, False)(_as_u8(src) if not isinstance(src, torch.Tensor) else src, h, w, c)


def _to_float(src, layout: str, normalize: bool, dtype):
    """Image or uint8 tensor -> [H, W, C] floating tensor (values / 255 with ``normalize``). With
    ``layout="CHW"`` the source's axes are read as (C, H, W) the way the reference does, i.e. the result keeps
    the source's element order and only its interpretation changes."""
    t = src.data if hasattr(src, "meta") else src
    if t.dim() == 2:
        t = t[..., None]
    elif t.dim() == 1:
        t = t[:, None, None]
    out = t.to(dtype)
    return out / 255.0 if normalize else out


def to_tensor_float64(src, layout: str = "HWC", normalize: bool = True):
    """legacy/src/momijo/vision/convert.mojo:41-76"""
    return _to_float(src, layout, normalize, torch.float64)


def to_tensor_float32(src, layout: str = "HWC", normalize: bool = True):
    """legacy/src/momijo/vision/convert.mojo:100-135"""
    return _to_float(src, layout, normalize, torch.float32)
