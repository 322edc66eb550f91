"""Imports written against the reference's file layout resolve: consolidated packages serve the reference's module
paths as facades, and a name the reference keeps in another file of a package is still found there."""
import importlib

import pytest


@pytest.mark.parametrize("path,name", [
    ("momijo.dataframe.series_bool", "SeriesBool"), ("momijo.dataframe.bitmap", "Bitmap"),
    ("momijo.dataframe.join", "append_row"), ("momijo.dataframe._groupby_core", "Agg"),
    ("momijo.vision.io.huffman", "HuffmanTable"), ("momijo.vision.io.inflate", "BitReader"),
    ("momijo.vision.backend.cpu.simd.resize_simd_u8_hwc", "resize_u8_hwc_nearest_simd"),
    ("momijo.vision.schedule", "auto_schedule"), ("momijo.vision.transforms.features", "Keypoint"),
    ("momijo.visual.charts.ez_option", "EasyOption"), ("momijo.visual.core.core", "echarts_html"),
    ("momijo.visual.misc.marching_squares", "marching_squares"), ("momijo.learn.optim.sgd", "ReduceLROnPlateau"),
    ("momijo.learn.utils.summary", "MinMaxObserver"), ("momijo.tensor.helpers", "write_planeT"),
])
def test_reference_path_resolves(path, name):
    mod = importlib.import_module(path)
    obj = getattr(mod, name)
    assert obj is not None and importlib.import_module(path.replace("momijo.", "momijo_b200.", 1)) is mod


def test_unknown_names_still_fail():
    mod = importlib.import_module("momijo.dataframe.series_bool")
    with pytest.raises(AttributeError):
        mod.no_such_name
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("momijo.dataframe.no_such_module")
