"""Byte buffers, typed views and copy helpers (legacy/src/momijo/vision/memory.mojo:11-420).

The reference hands out raw pointers; here an allocation is a one-dimensional torch tensor on the host
(``alloc_*`` uninitialised, ``calloc_*`` zeroed), which plays the pointer's part in the ``mem*`` helpers: they
take tensors (or ``memoryview``-compatible objects) and optional element offsets. ``free_*`` exist for source
compatibility and do nothing (the tensor's memory goes when its last reference does). ``ViewU8`` is a
non-owning window, ``BufferU8`` an owning byte buffer; the ``as_*_view`` functions reinterpret a buffer's
bytes without copying."""
from __future__ import annotations

import torch


def _alloc(n: int, dt, zero: bool) -> torch.Tensor:
    n = max(int(n), 0)
    return torch.zeros(n, dtype=dt) if zero else torch.empty(n, dtype=dt)


def alloc_u8(nbytes: int): return _alloc(nbytes, torch.uint8, False)      # noqa: E704
def calloc_u8(nbytes: int): return _alloc(nbytes, torch.uint8, True)      # noqa: E704
def alloc_u16(nelems: int): return _alloc(nelems, torch.uint16, False)    # noqa: E704
def calloc_u16(nelems: int): return _alloc(nelems, torch.uint16, True)    # noqa: E704
def alloc_i32(nelems: int): return _alloc(nelems, torch.int32, False)     # noqa: E704
def calloc_i32(nelems: int): return _alloc(nelems, torch.int32, True)     # noqa: E704
def alloc_i64(nelems: int): return _alloc(nelems, torch.int64, False)     # noqa: E704
def calloc_i64(nelems: int): return _alloc(nelems, torch.int64, True)     # noqa: E704
def alloc_f32(nelems: int): return _alloc(nelems, torch.float32, False)   # noqa: E704
def calloc_f32(nelems: int): return _alloc(nelems, torch.float32, True)   # noqa: E704
def alloc_f64(nelems: int): return _alloc(nelems, torch.float64, False)   # noqa: E704
def calloc_f64(nelems: int): return _alloc(nelems, torch.float64, True)   # noqa: E704


def _free(ptr) -> None:
    return None


free_u8 = free_u16 = free_i32 = free_i64 = free_f32 = free_f64 = _free


def _u8(x) -> torch.Tensor:
    if isinstance(x, (ViewU8, BufferU8)):
        return x.data()
    if isinstance(x, torch.Tensor):
        return x.reshape(-1).view(torch.uint8) if x.dtype != torch.uint8 else x.reshape(-1)
    return torch.frombuffer(x if not isinstance(x, bytes) else bytearray(x), dtype=torch.uint8)


def memcpy_u8(dst, src, nbytes: int) -> None:
    if nbytes > 0:
        _u8(dst)[:nbytes] = _u8(src)[:nbytes]


def memmove_u8(dst, src, nbytes: int) -> None:
    """Copy that is correct for overlapping ranges."""
    if nbytes > 0:
        _u8(dst)[:nbytes] = _u8(src)[:nbytes].clone()


def memset_u8(dst, value: int, nbytes: int) -> None:
    if nbytes > 0:
        _u8(dst)[:nbytes] = int(value) & 255


def memcmp_u8(a, b, nbytes: int) -> int:
    """0 when equal, else the difference of the first differing bytes (a - b)."""
    x, y = _u8(a)[:nbytes].to(torch.int16), _u8(b)[:nbytes].to(torch.int16)
    d = (x != y).nonzero()
    if d.numel() == 0:
        return 0
    i = int(d[0])
    return int(x[i] - y[i])


def pointer_add_u8(p, offset_bytes: int):
    """The same bytes from ``offset_bytes`` on (a view)."""
    return _u8(p)[offset_bytes:]


def hexdigit(n: int) -> int:
    n = int(n) & 15
    return ord("0") + n if n < 10 else ord("A") + n - 10


def byte_to_hex(b: int) -> str:
    return chr(hexdigit((int(b) >> 4) & 15)) + chr(hexdigit(int(b) & 15))


def hexdump_head(p, nbytes: int, maxn: int) -> str:
    k = min(max(maxn, 0), nbytes)
    return " ".join(byte_to_hex(v) for v in _u8(p)[:k].tolist())


def hexdump_full(p, nbytes: int) -> str:
    vals = _u8(p)[:nbytes].tolist()
    return "\n".join(" ".join(byte_to_hex(v) for v in vals[i:i + 16]) for i in range(0, len(vals), 16))


class ViewU8:
    """Non-owning window of ``length_bytes`` bytes."""

    def __init__(self, data=None, length_bytes: int = 0):
        t = _u8(data) if data is not None else torch.zeros(0, dtype=torch.uint8)
        n = min(max(length_bytes, 0), t.numel())
        self._data = t[:n]

    def data(self) -> torch.Tensor:
        return self._data

    def length(self) -> int:
        return self._data.numel()

    def is_empty(self) -> bool:
        return self._data.numel() == 0

    def slice(self, offset: int, size: int) -> "ViewU8":
        off, sz = max(offset, 0), max(size, 0)
        if off >= self.length():
            return ViewU8(None, 0)
        return ViewU8(self._data[off:], min(sz, self.length() - off))


class BufferU8:
    """Owning byte buffer; ``copy`` / ``clone`` duplicate the bytes, ``view`` / ``slice`` share them."""

    def __init__(self, length_bytes: int = 0, zero_init: bool = False):
        self._data = calloc_u8(length_bytes) if zero_init else alloc_u8(length_bytes)

    def copy(self) -> "BufferU8":
        out = BufferU8(0)
        out._data = self._data.clone()
        return out

    clone = copy

    def data(self) -> torch.Tensor:
        return self._data

    def length(self) -> int:
        return self._data.numel()

    def view(self) -> ViewU8:
        return ViewU8(self._data, self.length())

    def zero(self) -> None:
        self._data.zero_()

    def fill(self, value: int) -> None:
        self._data.fill_(int(value) & 255)

    def slice(self, offset: int, size: int) -> ViewU8:
        return self.view().slice(offset, size)

    def _clip(self, off: int, n: int) -> int:
        if off < 0 or n <= 0 or off >= self.length():
            return 0
        return min(n, self.length() - off)

    def write_from(self, src, nbytes: int, dst_offset: int = 0) -> None:
        n = self._clip(dst_offset, nbytes)
        if n:
            self._data[dst_offset:dst_offset + n] = _u8(src)[:n]

    def read_into(self, dst, nbytes: int, src_offset: int = 0) -> None:
        n = self._clip(src_offset, nbytes)
        if n:
            _u8(dst)[:n] = self._data[src_offset:src_offset + n]

    def copy_range(self, src_offset: int, dst_offset: int, nbytes: int) -> None:
        """Overlap-safe move inside the buffer; out-of-range requests are clipped."""
        n = min(self._clip(src_offset, nbytes), self._clip(dst_offset, nbytes))
        if n:
            self._data[dst_offset:dst_offset + n] = self._data[src_offset:src_offset + n].clone()


def _typed(buf: BufferU8, nelems: int, dt) -> torch.Tensor:
    size = torch.empty(0, dtype=dt).element_size()
    if nelems <= 0 or nelems * size > buf.length():
        return torch.zeros(0, dtype=dt)
    return buf.data()[: nelems * size].view(dt)


def as_u16_view(buf: BufferU8, nelems: int): return _typed(buf, nelems, torch.uint16)    # noqa: E704
def as_i32_view(buf: BufferU8, nelems: int): return _typed(buf, nelems, torch.int32)     # noqa: E704
def as_i64_view(buf: BufferU8, nelems: int): return _typed(buf, nelems, torch.int64)     # noqa: E704
def as_f32_view(buf: BufferU8, nelems: int): return _typed(buf, nelems, torch.float32)   # noqa: E704
def as_f64_view(buf: BufferU8, nelems: int): return _typed(buf, nelems, torch.float64)   # noqa: E704


def copy_bytes_to_new(src, nbytes: int) -> BufferU8:
    out = BufferU8(max(nbytes, 0))
    out.write_from(src, nbytes, 0)
    return out


def copy_buffer(src: BufferU8) -> BufferU8:
    return src.copy()
