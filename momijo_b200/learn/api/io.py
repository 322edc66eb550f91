"""``save_model / load_model / load_into`` with the default ``.mnp`` extension and best-effort
parent ``mkdir`` (legacy/src/momijo/learn/api/io.mojo:35-143)."""
from __future__ import annotations

import os

from ..utils.checkpoint import load_state_dict, save_state_dict


def _normalize_and_default_ext(path: str) -> str:
    last = os.path.basename(path)
    return path + ".mnp" if "." not in last else path


def _ensure_parent_dir(path: str):
    d = os.path.dirname(path)
    if d:
        try:
            os.makedirs(d, exist_ok=True)
        except OSError:
            pass


def save_model_ok(model, path: str) -> bool:
    p = _normalize_and_default_ext(path)
    _ensure_parent_dir(p)
    try:
        save_state_dict(getattr(model, "net", model), p)
        return True
    except OSError:
        return False


def save_model(model, path: str):
    save_model_ok(model, path)


def load_into(model, path: str) -> bool:
    return load_state_dict(getattr(model, "net", model), _normalize_and_default_ext(path))


def load_model_ok(path: str):
    from .model import Model

    m = Model()
    return os.path.exists(_normalize_and_default_ext(path) + ".json"), m


def load_model(path: str):
    return load_model_ok(path)[1]


load_new = load_model_ok
