"""The vision package's own small tensor type is a strided raw pointer in the reference
(legacy/src/momijo/vision/tensor.mojo:35); here it is a torch tensor, and this module keeps the
helper names that code written against the reference imports."""
from __future__ import annotations

import torch

Tensor = torch.Tensor


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
