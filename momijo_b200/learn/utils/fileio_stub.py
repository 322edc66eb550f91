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
