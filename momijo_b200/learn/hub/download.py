"""``cached_download`` with FNV-1a / SHA-256 verification; ``file://`` and plain paths only, HTTP is
a hook (legacy/src/momijo/learn/hub/download.mojo:26-379; there is no network on the build
machines either)."""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
from dataclasses import dataclass

from ... import _C


@dataclass
class DownloadOptions:
    cache_enabled: bool = True
    retries: int = 2
    timeout_sec: int = 60
    allow_resume: bool = True
    expected_fnv64: str = ""
    expected_sha256: str = ""
    user_agent: str = "MomijoLearn/0.1"


http_hook = None  # callable(url, tmp_path, opts) -> bool, installed by the application


def _fnv1a64(data: bytes) -> str:
    try:
        h = _C.host()
        h.mmj_fnv1a64.argtypes = [ctypes.c_char_p, ctypes.c_longlong]
        h.mmj_fnv1a64.restype = ctypes.c_ulonglong
        return f"{h.mmj_fnv1a64(data, len(data)):016x}"
    except Exception:
        v = 1469598103934665603
        for b in data:
            v = ((v ^ b) * 1099511628211) & ((1 << 64) - 1)
        return f"{v:016x}"


def _sha256(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def _verify_checksums(data: bytes, opts: DownloadOptions) -> bool:
    if opts.expected_fnv64 and _fnv1a64(data) != opts.expected_fnv64.lower():
        return False
    if opts.expected_sha256 and _sha256(data) != opts.expected_sha256.lower():
        return False
    return True


def _basename_from_url(url: str) -> str:
    b = url.split("?")[0].rstrip("/").rsplit("/", 1)[-1]
    return b or "download.bin"


def cached_download(url: str, path: str, opts: DownloadOptions | None = None) -> str:
    """Fetch ``url`` into ``path`` (a file, or a directory to which the URL's basename is added);
    returns the final path, or "" on failure."""
    opts = opts or DownloadOptions()
    dst = os.path.join(path, _basename_from_url(url)) if (os.path.isdir(path) or path.endswith(os.sep)) else path
    if opts.cache_enabled and os.path.exists(dst):
        with open(dst, "rb") as f:
            if _verify_checksums(f.read(), opts):
                return dst
    os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
    tmp = dst + ".part"
    ok = False
    for _ in range(max(1, opts.retries + 1)):
        try:
            if url.startswith("file://") or os.path.exists(url):
                shutil.copyfile(url[7:] if url.startswith("file://") else url, tmp)
                ok = True
            elif http_hook is not None:
                ok = bool(http_hook(url, tmp, opts))
        except OSError:
            ok = False
        if ok:
            break
    if not ok:
        return ""
    with open(tmp, "rb") as f:
        data = f.read()
    if not _verify_checksums(data, opts):
        os.remove(tmp)
        return ""
    os.replace(tmp, dst)
    return dst
