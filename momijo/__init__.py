"""``momijo`` import name: code written against the reference's package layout
(``momijo.tensor``, ``momijo.learn``, ``momijo.dataframe``, ``momijo.vision``, ``momijo.visual``;
legacy/src/momijo/__init__.mojo) resolves to the modules of ``momijo_b200``. Every ``momijo.x.y`` is
the very same module object as ``momijo_b200.x.y``, so state (registries, default process group, kernel
library handle) is shared whichever name is used."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import momijo_b200 as _impl

_PREFIX = __name__ + "."
_TARGET = _impl.__name__ + "."


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            mod = importlib.import_module(real)
        except ModuleNotFoundError as e:
            if e.name == real:
                return None
            raise
        spec = importlib.util.spec_from_loader(fullname, self, is_package=hasattr(mod, "__path__"))
        spec._momijo_real = mod
        return spec

    def create_module(self, spec):
        return spec._momijo_real

    def exec_module(self, module):
        return None


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__version__ = getattr(_impl, "__version__", "0")


def __getattr__(name):
    try:
        return importlib.import_module(_PREFIX + name)
    except ModuleNotFoundError:
        return getattr(_impl, name)
