"""``save_checkpoint_files`` / ``load_checkpoint_files``
(legacy/src/momijo/learn/utils/checkpoint_fileio.mojo:88-114): header text + CSV "blob"."""
import os

import torch

from .checkpoint import make_checkpoint, apply_checkpoint
from .tensor_bytes import pack_f64_to_bytes, unpack_bytes_to_f64


def save_checkpoint_files(net, header_path: str, blob_path: str) -> bool:
    try:
        header, flat = make_checkpoint(net)
        with open(header_path, "w") as f:
            f.write(header)
        with open(blob_path, "wb") as f:
            f.write(pack_f64_to_bytes(flat).numpy().tobytes())
        return True
    except OSError:
        return False


def load_checkpoint_files(header_path, blob_path: str = None, blob_path_ref: str = None):
    """``load_checkpoint_files(header_path, blob_path)`` -> (ok, header, blob tensor); the reference's
    ``load_checkpoint_files(net, header_path, blob_path)`` loads into ``net`` and returns whether that worked
    (legacy/src/momijo/learn/utils/checkpoint_fileio.mojo:102-114)."""
    if blob_path_ref is not None:
        return load_into(header_path, blob_path, blob_path_ref)
    if not (os.path.exists(header_path) and os.path.exists(blob_path)):
        return False, "", torch.zeros(0)
    with open(header_path) as f:
        header = f.read()
    with open(blob_path, "rb") as f:
        blob = unpack_bytes_to_f64(f.read())
    return True, header, blob


def load_into(net, header_path: str, blob_path: str) -> bool:
    ok, header, blob = load_checkpoint_files(header_path, blob_path)
    return ok and apply_checkpoint(net, header, blob)
