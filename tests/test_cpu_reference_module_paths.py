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


def test_reference_call_forms():
    """Longer argument lists of the reference are accepted next to this package's own forms."""
    import torch

    import momijo.dataframe as D
    import momijo.tensor as mt
    from momijo.learn.losses import regression as RG
    from momijo.learn.nn import functional as F
    from momijo.tensor import axis as AX, errors as E, io as IO, transform as TR
    x = torch.arange(32.0).reshape(1, 2, 4, 4)
    assert torch.equal(F.im2col(x, (3, 3), 1, 0), F.im2col(x, 3, 3, 1, 0))
    assert F.max_pool2d([[[[1.0, 2.0], [3.0, 4.0]]]], 2, 0) == [[[[4.0]]]]
    assert RG.mse_loss([1.0, 3.0], [0.0, 0.0], "mean", [1.0, 3.0]) == 7.0
    t = mt.from_list([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    assert AX.quantile(t, 0.5, axes=[0, 1]).item() == 3.5 and AX.median(t, axes=[1]).tolist() == [2.0, 5.0]
    assert not E.check_axis(2, 2) and E.check_axis(1, 2) and not E.check_same_shape([2, 3], [2, 4])
    assert TR.pad_nd_map(mt.from_list([1, 2, 3]), [1, 1], 4, 9).tolist() == [9, 1, 2, 3, 9]
    assert IO.csv_to_tensor_with(IO.tensor_to_csv(t)).tolist() == t.tolist()
    assert D.int64(True).is_nullable() and D.int64() == D.DType("int64")
    df = D.ToDataFrame({"d": ["2025-01-02", "x"], "c": ["lo", "hi"]}, ["r0", "r1"])
    assert df.index.labels == ["r0", "r1"] and D.datetime_year(df, "d", 2) == "2025-01-02, "
    assert D.to_category(df, "c", "k", False, ["hi"]).col("k").values == [-1, 0]
