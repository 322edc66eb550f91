"""In-memory model registry (legacy/src/momijo/learn/hub/registry.mojo:61-119)."""
from __future__ import annotations

_REG = {}


def register_model(name: str, constructor_path: str) -> bool:
    if not name or name in _REG:
        return False
    _REG[name] = constructor_path
    return True


def has_model(name: str) -> bool:
    return name in _REG


def get_constructor_path(name: str) -> str:
    return _REG.get(name, "")


def list_models():
    return sorted(_REG)


def unregister_model(name: str) -> bool:
    return _REG.pop(name, None) is not None


def clear_registry() -> int:
    n = len(_REG)
    _REG.clear()
    return n


def dump_registry():
    names = sorted(_REG)
    return names, [_REG[n] for n in names]


def build_model(name: str, *args, **kw):
    """Import ``pkg.module:attr`` or ``pkg.module.attr`` and call it."""
    import importlib

    path = _REG[name]
    mod, _, attr = path.partition(":") if ":" in path else path.rpartition(".")[::2] and (path.rpartition(".")[0], ".", path.rpartition(".")[2])
    return getattr(importlib.import_module(mod), attr)(*args, **kw)
