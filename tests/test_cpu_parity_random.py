"""Randomised parity checks (fixed seeds): tensor operations against NumPy, data-frame operations against pandas.
The reference's NumPy-parity demos fix single cases; these walk random shapes, axes and missing cells."""
import numpy as np
import pytest
import torch

import momijo_b200.dataframe as D
import momijo_b200.tensor as T
from momijo_b200.tensor import Tensor
from momijo_b200.tensor import nanops as N


def _mk(a):
    return Tensor(torch.from_numpy(np.ascontiguousarray(a)))


def _same(got, want):
    g = got.detach().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    want = np.asarray(want)
    assert g.shape == want.shape, (g.shape, want.shape)
    assert np.allclose(g.astype(np.float64), want.astype(np.float64), equal_nan=True)


@pytest.mark.parametrize("seed", range(12))
def test_tensor_ops_match_numpy(seed):
    rng = np.random.default_rng(seed)
    nd = int(rng.integers(1, 4))
    shape = tuple(int(v) for v in rng.integers(1, 6, size=nd))
    a = rng.standard_normal(shape)
    x = _mk(a)
    ax = int(rng.integers(-nd, nd))
    _same(T.roll(x, 2, ax), np.roll(a, 2, ax))
    _same(T.flip(x, ax), np.flip(a, ax))
    _same(T.cumsum(x, ax), np.cumsum(a, ax))
    _same(T.cumprod(x, ax), np.cumprod(a, ax))
    _same(T.swapaxes(x, 0, ax), np.swapaxes(a, 0, ax))
    _same(T.moveaxis(x, 0, ax), np.moveaxis(a, 0, ax))
    _same(T.tile(x, [2] * nd), np.tile(a, [2] * nd))
    _same(T.clip(x, -0.5, 0.5), np.clip(a, -0.5, 0.5))
    _same(T.mean(x, ax), np.mean(a, ax))
    _same(T.median(x, ax), np.median(a, ax))
    _same(T.quantile(x, 0.3, ax), np.quantile(a, 0.3, ax))
    _same(T.percentile(x, 70.0, ax), np.percentile(a, 70.0, ax))
    _same(T.unsqueeze(x, ax), np.expand_dims(a, ax))
    idx = rng.integers(0, shape[ax], size=3)
    _same(T.take(x, _mk(idx.astype(np.int64)), ax), np.take(a, idx, ax))
    order = np.argsort(a, axis=ax)
    _same(T.take_along_axis(x, _mk(order.astype(np.int64)), ax), np.take_along_axis(a, order, ax))
    _same(T.where(_mk(a > 0), x, _mk(np.zeros_like(a))), np.where(a > 0, a, 0))
    _same(x.sum(ax), a.sum(ax))
    _same(x.argmax(ax), a.argmax(ax))
    c = rng.standard_normal(shape[-1:])
    _same(x + _mk(c), a + c)
    _same(x * 2.5 - 1, a * 2.5 - 1)
    b = a.copy()
    b.flat[0] = np.nan
    _same(N.nansum(_mk(b), ax), np.nansum(b, ax))
    _same(N.nan_to_num(_mk(b)), np.nan_to_num(b))
    for sl in (slice(None, None, -1), slice(0, None, 2)):
        _same(x[sl], a[sl])
        w, y = a.copy(), _mk(a.copy())
        w[sl] = 7.0
        y[sl] = 7.0
        _same(y, w)
    if nd == 2:
        _same(T.tril(x), np.tril(a))
        _same(T.triu(x, 1), np.triu(a, 1))
        d = rng.standard_normal(shape[::-1])
        _same(T.tensordot(x, _mk(d), 1), np.tensordot(a, d, 1))
        for mode, npmode in (("constant", "constant"), ("symmetric", "symmetric"), ("replicate", "edge"),
                             ("circular", "wrap")):
            _same(T.pad(x, [(1, 1), (1, 1)], mode), np.pad(a, [(1, 1), (1, 1)], mode=npmode))
        if min(shape) >= 2:
            _same(T.pad(x, [(1, 1), (1, 1)], "reflect"), np.pad(a, [(1, 1), (1, 1)], mode="reflect"))


@pytest.mark.parametrize("seed", range(8))
def test_dataframe_ops_match_pandas(seed):
    pd = pytest.importorskip("pandas")
    rng = np.random.default_rng(100 + seed)
    n = int(rng.integers(3, 12))
    a = rng.integers(0, 5, n).tolist()
    b = [None if rng.random() < 0.2 else float(np.round(v, 3)) for v in rng.standard_normal(n)]
    k = [str(v) for v in rng.choice(list("xyz"), n)]
    df, pdf = D.DataFrame({"a": a, "b": b, "k": k}), pd.DataFrame({"a": a, "b": b, "k": k})

    got, want = df.sort_values("a").to_dict(), pdf.sort_values("a", kind="stable").to_dict(orient="list")
    assert got["a"] == want["a"] and got["k"] == want["k"]
    got, want = df.drop_duplicates(["a", "k"]).to_dict(), pdf.drop_duplicates(["a", "k"]).to_dict(orient="list")
    assert got["a"] == want["a"] and got["k"] == want["k"]

    got = D.groupby(df, "k", {"a": ["sum", "mean"], "b": ["mean", "count", "min", "max"]}).to_dict()
    w = pdf.groupby("k", sort=False).agg(a_sum=("a", "sum"), a_mean=("a", "mean"), b_mean=("b", "mean"),
                                         b_count=("b", "count"), b_min=("b", "min"), b_max=("b", "max"))
    assert got["k"] == list(w.index)          # groups in order of first appearance
    for c in (c for c in got if c != "k"):
        wc = [x for x in w.columns if x.replace("_", "") == c.replace("_", "")][0]
        gv = [np.nan if v is None else float(v) for v in got[c]]
        assert np.allclose(gv, w[wc].astype(float).tolist(), equal_nan=True), c

    right, pright = D.DataFrame({"k": ["x", "y"], "w": [10, 20]}), pd.DataFrame({"k": ["x", "y"], "w": [10, 20]})
    none = lambda v: None if v is None or (isinstance(v, float) and v != v) else int(v)
    for how in ("inner", "left"):
        got = df.merge(right, on="k", how=how).to_dict()
        want = pdf.merge(pright, on="k", how=how).to_dict(orient="list")
        assert sorted(zip(got["a"], got["k"], [str(none(v)) for v in got["w"]])) == \
            sorted(zip(want["a"], want["k"], [str(none(v)) for v in want["w"]])), how
