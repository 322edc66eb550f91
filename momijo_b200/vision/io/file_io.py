"""Byte-level file helpers and an in-memory file store (legacy/src/momijo/vision/io/file_io.mojo:116-400).

``MemFileStore`` maps path strings to byte strings (tests and pipelines that must not touch the disk write
their encoded images there). The ``memfs_*`` functions keep the reference's uniform result shape
``(ok, size, bytes, names, dummy)``; ``dummy`` stood for a raw pointer there and is always ``None`` here."""
from __future__ import annotations

import os
from typing import List, Tuple


class MemFileStore:
    def __init__(self):
        self.keys: List[str] = []
        self.vals: List[bytearray] = []

    def find(self, path: str) -> int:
        try:
            return self.keys.index(path)
        except ValueError:
            return -1

    def ensure(self, path: str) -> int:
        idx = self.find(path)
        if idx >= 0:
            return idx
        self.keys.append(path)
        self.vals.append(bytearray())
        return len(self.keys) - 1

    def write(self, path: str, data) -> int:
        idx = self.ensure(path)
        self.vals[idx] = bytearray(data)
        return len(self.vals[idx])

    def append(self, path: str, raw, n: int = None) -> int:
        idx = self.ensure(path)
        chunk = bytes(raw)
        self.vals[idx] += chunk if n is None else chunk[:n]
        return len(self.vals[idx])

    def size(self, path: str) -> int:
        idx = self.find(path)
        return 0 if idx < 0 else len(self.vals[idx])

    def read(self, path: str) -> bytes:
        idx = self.find(path)
        return b"" if idx < 0 else bytes(self.vals[idx])

    def remove(self, path: str) -> bool:
        """Swap-remove: the last entry takes the removed one's slot."""
        idx = self.find(path)
        if idx < 0:
            return False
        self.keys[idx], self.vals[idx] = self.keys[-1], self.vals[-1]
        self.keys.pop()
        self.vals.pop()
        return True

    def list(self) -> List[str]:
        return list(self.keys)

    def clear(self) -> int:
        n = len(self.keys)
        self.keys, self.vals = [], []
        return n


Result = Tuple[bool, int, bytes, List[str], None]


def memfs_try_read(fs: MemFileStore, path: str) -> Result:
    data = fs.read(path)
    return (len(data) > 0 or fs.find(path) >= 0, len(data), data, [], None)


def memfs_write_replace(fs: MemFileStore, path: str, data) -> Result:
    return (True, fs.write(path, data), b"", [], None)


def memfs_append_ptr(fs: MemFileStore, path: str, raw, n: int) -> Result:
    return (True, fs.append(path, raw, n), b"", [], None)


def memfs_size_of(fs: MemFileStore, path: str) -> Result:
    sz = fs.size(path)
    return (sz > 0 or fs.find(path) >= 0, sz, b"", [], None)


def memfs_remove_path(fs: MemFileStore, path: str) -> Result:
    return (fs.remove(path), 0, b"", [], None)


def memfs_list_all(fs: MemFileStore) -> Result:
    names = fs.list()
    return (True, len(names), b"", names, None)


def memfs_clear_all(fs: MemFileStore) -> Result:
    return (True, fs.clear(), b"", [], None)


def memfs_has_path(fs: MemFileStore, path: str) -> Result:
    return (fs.find(path) >= 0, 0, b"", [], None)


def memfs_ensure_path(fs: MemFileStore, path: str) -> Result:
    return (fs.ensure(path) >= 0, 0, b"", [], None)


def read_all_bytes(path: str) -> bytes:
    """The file's bytes; raises OSError when it cannot be read."""
    with open(path, "rb") as f:
        return f.read()


def write_all_bytes(path: str, data) -> bool:
    """Writes ``data`` (bytes or a list of ints), creating the parent directory; raises OSError on failure."""
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "wb") as f:
        f.write(bytes(data))
    return True


def ensure_outdir(path: str) -> bool:
    """Make sure the parent directory of ``path`` exists (legacy/src/momijo/vision/io/image.mojo:48-64)."""
    parent = os.path.dirname(path)
    if not parent:
        return True
    try:
        os.makedirs(parent, exist_ok=True)
        return True
    except OSError:
        return False
