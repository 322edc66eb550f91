"""Module paths of the reference that this package serves from fewer, larger modules.

The reference spreads ``dataframe``, ``vision`` and ``visual`` over many small files (``dataframe/series_bool.mojo``,
``vision/io/huffman.mojo``, ``visual/charts/ez_option.mojo`` ...); here each of those packages keeps its code in a
handful of modules. So that ``from momijo.dataframe.series_bool import SeriesBool`` keeps working, every reference
module path listed below imports as a facade: a module object whose attributes resolve, on first use, to the objects
of the same name in the enclosing modules of this package (nearest parent first, then the package's other modules).
No code lives in a facade, and a name the package does not define raises ``AttributeError`` as usual.
``tensor`` and ``learn`` need no facades: their module layout already matches the reference's."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys
import types

_ROOT = __name__.rsplit(".", 1)[0]

FACADES = (
    # dataframe
    "dataframe._groupby_core", "dataframe.api", "dataframe.bitmap", "dataframe.categorical", "dataframe.column",
    "dataframe.compat", "dataframe.datetime_ops", "dataframe.encoding", "dataframe.exec", "dataframe.helpers",
    "dataframe.io_bytes", "dataframe.io_csv", "dataframe.io_facade", "dataframe.io_json_min",
    "dataframe.io_pickle_mnp", "dataframe.join", "dataframe.missing", "dataframe.multiindex", "dataframe.query",
    "dataframe.selection", "dataframe.series", "dataframe.series_bool", "dataframe.series_f64",
    "dataframe.series_i64", "dataframe.series_str", "dataframe.stats_core", "dataframe.string_ops",
    "dataframe.utils",
    # vision
    "vision.adapters.arrow", "vision.backend.cpu.convert_color_cpu", "vision.backend.cpu.resize_cpu",
    "vision.backend.cpu.resize_tiled_cpu", "vision.backend.cpu.simd.convert_simd_u8_hwc",
    "vision.backend.cpu.simd.resize_simd_u8_hwc", "vision.convert", "vision.io.bitreader", "vision.io.bitwriter",
    "vision.io.color_ycbcr", "vision.io.decode_jpeg", "vision.io.decode_png", "vision.io.encode_jpeg",
    "vision.io.encode_png", "vision.io.huffman", "vision.io.idct", "vision.io.image_read", "vision.io.image_write",
    "vision.io.inflate", "vision.io.jpeg_dct", "vision.io.jpeg_decoder", "vision.io.jpeg_huffman_encode",
    "vision.io.jpeg_quantize", "vision.io.jpeg_scan", "vision.io.jpeg_writer", "vision.io.png_decoder",
    "vision.io.registry", "vision.io.tables", "vision.io.unfilter", "vision.transforms.convert_color",
    "vision.transforms.normalize", "vision.transforms.resize", "vision.transforms.tile",
    "vision.transforms.transforms",
    # visual
    "visual.charts.ez_option", "visual.charts.option", "visual.core.core", "visual.core.echarts_core",
    "visual.html.html_viewer", "visual.html.preview", "visual.misc.bar", "visual.misc.calendar",
    "visual.misc.candlestick", "visual.misc.custom", "visual.misc.dashboard", "visual.misc.effectscatter",
    "visual.misc.export", "visual.misc.funnel", "visual.misc.gauge", "visual.misc.heatmap", "visual.misc.histogram",
    "visual.misc.kde", "visual.misc.line", "visual.misc.lines", "visual.misc.map", "visual.misc.marching_squares",
    "visual.misc.parallel", "visual.misc.pictorialbar", "visual.misc.pie", "visual.misc.radar",
    "visual.misc.registry", "visual.misc.sankey", "visual.misc.scatter", "visual.misc.sunburst",
    "visual.misc.themeriver", "visual.misc.themes", "visual.misc.treemap", "visual.misc.types",
    "visual.plotting.boxplot", "visual.plotting.echarts_3d", "visual.plotting.echarts_axes",
    "visual.plotting.echarts_custom", "visual.plotting.echarts_exporter", "visual.plotting.echarts_layout",
    "visual.plotting.echarts_polar", "visual.plotting.echarts_sankey", "visual.plotting.echarts_series",
    "visual.plotting.graph", "visual.plotting.violin_utils",
)
# reference directories that hold facade modules and are not packages (or not even modules) here
FACADE_PACKAGES = ("visual.charts", "vision.adapters", "vision.backend.cpu.simd", "vision.schedule")
# modules of this package that stand where the reference has a directory: they accept facade submodules
MODULES_WITH_SUBMODULES = ("visual.core", "visual.html", "visual.misc", "visual.plotting")


def _resolver(rel: str):
    parts = rel.split(".")
    parents = [_ROOT + "." + ".".join(parts[:k]) for k in range(len(parts) - 1, 0, -1)]
    package = _ROOT + "." + parts[0]

    def lookup(name: str):
        if name.startswith("__") or name == "_momijo_facade":
            raise AttributeError(name)
        for modname in parents:
            mod = sys.modules.get(modname)
            if mod is not None and not vars(mod).get("_momijo_facade", False) and name in vars(mod):
                return vars(mod)[name]
        for modname, mod in list(sys.modules.items()):
            if modname.startswith(package + ".") and mod is not None and not vars(mod).get("_momijo_facade", False) \
                    and name in vars(mod):
                return vars(mod)[name]
        raise AttributeError(f"module {_ROOT}.{rel!s} has no attribute {name!r}")
    return lookup


class _FacadeFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ROOT + "."):
            return None
        rel = fullname[len(_ROOT) + 1:]
        if rel not in FACADES and rel not in FACADE_PACKAGES:
            return None
        return importlib.util.spec_from_loader(fullname, self, is_package=rel in FACADE_PACKAGES)

    def create_module(self, spec):
        rel = spec.name[len(_ROOT) + 1:]
        importlib.import_module(_ROOT + "." + rel.split(".")[0])          # the real package, so lookups can succeed
        mod = types.ModuleType(spec.name, f"Facade for the reference module path momijo.{rel}: names resolve to this "
                                           f"package's implementations.")
        mod._momijo_facade = True
        mod.__getattr__ = _resolver(rel)
        if rel in FACADE_PACKAGES:
            mod.__path__ = []
        return mod

    def exec_module(self, module):
        return None


def link_siblings(package: str) -> None:
    """Give every loaded module of ``package`` (a sub-package name such as ``"learn"``) a fallback attribute lookup
    into its enclosing modules and siblings. The reference sometimes defines a name in one file and this package in
    another (its ``optim/sgd.mojo`` also holds the schedulers; ``io/jpeg.mojo`` the functions kept here in
    ``io/image.py``); with the fallback, ``from momijo.learn.optim.sgd import StepLR`` finds it. Modules that already
    have their own module-level ``__getattr__`` are left alone."""
    import pkgutil
    prefix = _ROOT + "." + package
    pkg = sys.modules.get(prefix)
    if pkg is not None and getattr(pkg, "__file__", None):      # load the modules nothing has imported yet
        import os
        for info in pkgutil.walk_packages([os.path.dirname(pkg.__file__)], prefix + "."):
            if info.name not in sys.modules and ".gpu." not in info.name and not info.name.rsplit(".", 1)[-1].startswith("bench"):
                try:
                    importlib.import_module(info.name)
                except Exception:
                    pass
    for modname, mod in list(sys.modules.items()):
        if mod is None or not (modname == prefix or modname.startswith(prefix + ".")):
            continue
        if vars(mod).get("_momijo_facade", False) or "__getattr__" in vars(mod) or modname == prefix:
            continue
        mod.__getattr__ = _resolver(modname[len(_ROOT) + 1:])


def install() -> None:
    if not any(isinstance(f, _FacadeFinder) for f in sys.meta_path):
        sys.meta_path.append(_FacadeFinder())


def open_submodules() -> None:
    """Let the modules that stand where the reference has a directory accept facade submodules."""
    for rel in MODULES_WITH_SUBMODULES:
        mod = sys.modules.get(_ROOT + "." + rel)
        if mod is not None and not hasattr(mod, "__path__"):
            mod.__path__ = []
