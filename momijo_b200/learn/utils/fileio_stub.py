"""Best-effort text file helpers (legacy/src/momijo/learn/utils/fileio_stub.mojo)."""
import os


def write_text(path: str, s: str) -> bool:
    try:
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        with open(path, "w") as f:
            f.write(s)
        return True
    except OSError:
        return False


def read_text(path: str) -> str:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return ""


def exists(path: str) -> bool:
    return os.path.exists(path)


def write_all_bytes(path: str, data) -> bool:
    """Write a uint8 tensor (or bytes / list of ints) to ``path``; False on failure
    (legacy/src/momijo/learn/utils/fileio_stub.mojo:13-20, which goes through a text file; this one
    writes the bytes as they are)."""
    import torch
    try:
        if isinstance(data, (bytes, bytearray)):
            raw = bytes(data)
        else:
            if not isinstance(data, torch.Tensor):
                from ...tensor.tensor import _raw
                data = _raw(data) if hasattr(data, "shape") else torch.as_tensor(list(data))
            raw = data.detach().to("cpu", torch.uint8).contiguous().numpy().tobytes()
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        with open(path, "wb") as f:
            f.write(raw)
        return True
    except (OSError, ValueError, TypeError):
        return False


def read_all_bytes(path: str):
    """uint8 tensor with the file's bytes; an empty tensor if the file is missing or unreadable
    (legacy/src/momijo/learn/utils/fileio_stub.mojo:22-31)."""
    import torch
    try:
        with open(path, "rb") as f:
            raw = f.read()
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8) if raw else torch.zeros(0, dtype=torch.uint8)
    except OSError:
        return torch.zeros(0, dtype=torch.uint8)
