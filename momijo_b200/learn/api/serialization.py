"""Layout-B serialisation: ``save / load / load_into / save_linear / load_linear``
(legacy/src/momijo/learn/api/serialization.mojo:148-215): ``base.header.json`` + ``base.state.bin``
(ASCII CSV despite the name)."""
from __future__ import annotations

import os

import torch

from ..utils.checkpoint import apply_checkpoint
from ..utils.checkpoint_fileio import load_checkpoint_files, save_checkpoint_files
from ..utils.tensor_bytes import pack_f64_to_bytes, unpack_bytes_to_f64


def _header_path(base):
    return base + ".header.json"


def _blob_path(base):
    return base + ".state.bin"


def save(net, base: str) -> bool:
    return save_checkpoint_files(net, _header_path(base), _blob_path(base))


def load(base: str):
    return load_checkpoint_files(_header_path(base), _blob_path(base))


def load_state_dict(net, header: str, blob: torch.Tensor) -> bool:
    return apply_checkpoint(net, header, blob)


def load_into(net, base: str) -> bool:
    ok, header, blob = load(base)
    return ok and apply_checkpoint(net, header, blob)


def save_linear(m, base: str) -> bool:
    try:
        with open(_header_path(base), "w") as f:
            f.write('{"type":"Linear","in":%d,"out":%d}' % (m.in_features, m.out_features))
        flat = torch.cat([m.weight.detach().float().reshape(-1), m.bias_t.detach().float().reshape(-1)])
        with open(_blob_path(base), "wb") as f:
            f.write(pack_f64_to_bytes(flat).numpy().tobytes())
        return True
    except OSError:
        return False


def load_linear(base: str):
    return load(base)


def load_state_dict_linear(m, blob: torch.Tensor) -> bool:
    nW, nB = m.weight.numel(), m.bias_t.numel()
    if blob.numel() < nW + nB:
        return False
    with torch.no_grad():
        m.weight.copy_(blob[:nW].view_as(m.weight).to(m.weight.dtype))
        m.bias_t.copy_(blob[nW:nW + nB].to(m.bias_t.dtype))
    return True
