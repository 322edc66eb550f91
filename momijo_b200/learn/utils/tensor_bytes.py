"""Float vector <-> ASCII CSV bytes (legacy/src/momijo/learn/utils/tensor_bytes.mojo:40-85): the
"binary" names are CSV in the reference too. Formatting/parsing runs in the C++ host runtime."""
from __future__ import annotations

import ctypes

import torch

from ... import _C


def _host():
    h = _C.host()
    h.mmj_pack_csv_f32.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_char_p, ctypes.c_longlong]
    h.mmj_pack_csv_f32.restype = ctypes.c_longlong
    h.mmj_unpack_csv_f32.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong]
    h.mmj_unpack_csv_f32.restype = ctypes.c_longlong
    return h


def pack_f64_to_bytes(x: torch.Tensor) -> torch.Tensor:
    """Float32 tensor -> uint8 tensor holding comma-separated decimals."""
    xf = x.detach().to(torch.float32).reshape(-1).contiguous().cpu()
    n = xf.numel()
    if n == 0:
        return torch.zeros(0, dtype=torch.uint8)
    h = _host()
    cap = n * 20 + 16
    buf = ctypes.create_string_buffer(cap)
    ln = h.mmj_pack_csv_f32(xf.data_ptr(), n, buf, cap)
    if ln < 0:
        buf = ctypes.create_string_buffer(-ln)
        ln = h.mmj_pack_csv_f32(xf.data_ptr(), n, buf, -ln)
    return torch.frombuffer(bytearray(buf.raw[:ln]), dtype=torch.uint8)


def unpack_bytes_to_f64(b) -> torch.Tensor:
    raw = bytes(b.cpu().numpy().tobytes()) if isinstance(b, torch.Tensor) else bytes(b)
    if not raw:
        return torch.zeros(0, dtype=torch.float32)
    h = _host()
    cap = raw.count(b",") + 1
    out = torch.empty(cap, dtype=torch.float32)
    n = h.mmj_unpack_csv_f32(raw, len(raw), out.data_ptr(), cap)
    return out[:n]


pack_f64_to_bytes_binary = pack_f64_to_bytes
unpack_bytes_to_f64_binary = unpack_bytes_to_f64
pack_f64 = pack_f64_to_bytes
unpack_f64 = unpack_bytes_to_f64
