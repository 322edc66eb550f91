"""DataFrame package: construction, selection, group-by / merge / pivot, missing data, windows, strings, I/O."""
import math

import momijo_b200.dataframe as D


def _df():
    p = D.make_pairs()
    p = D.pairs_append(p, "city", ["a", "b", "a", "c", "b", "a"]) or p
    p = D.pairs_append(p, "x", [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]) or p
    p = D.pairs_append(p, "n", [1, 2, 3, 4, 5, 6]) or p
    return D.df_from_pairs(p)


def _col(df, name):
    return list(df[name].values) if hasattr(df[name], "values") else list(df[name])


def test_construct_select_filter_sort():
    df = _df()
    assert D.df_shape(df) == (6, 3)
    assert D.df_shape(D.head(df, 2)) == (2, 3)
    f = D.filter(df, D.col_ge(df, "x", 4.0))
    assert _col(f, "n") == [4, 5, 6]
    s = D.sort_values(df, "x", ascending=False)
    assert _col(s, "n")[0] == 6
    sub = D.iloc(df, [0, 2], [0, 1])
    assert D.df_shape(sub) == (2, 2)
    assert D.df_shape(D.drop_duplicates(df, subset=["city"])) == (3, 3)


def test_groupby_merge_pivot_melt():
    df = _df()
    g = D.groupby(df, "city", [D.Agg("x", "sum", "sx"), D.Agg("n", "count", "cnt")])
    rows = {c: (s, k) for c, s, k in zip(_col(g, "city"), _col(g, "sx"), _col(g, "cnt"))}
    assert rows["a"] == (10.0, 3) and rows["b"] == (7.0, 2) and rows["c"] == (4.0, 1)
    right = D.DataFrame({"city": ["a", "b"], "pop": [10, 20]})
    m = D.merge(df, right, on="city", how="inner")
    assert D.df_shape(m)[0] == 5 and _col(m, "pop") == [10, 20, 10, 20, 10]
    ml = D.merge(df, right, on="city", how="left")
    assert D.df_shape(ml)[0] == 6
    pv = D.pivot_table(df, index="city", columns="n", values="x", aggfunc="sum", fill_value=0.0)
    assert D.df_shape(pv)[0] == 3
    long = D.melt(D.DataFrame({"id": [1, 2], "p": [3, 4], "q": [5, 6]}), id_vars=["id"])
    assert D.df_shape(long) == (4, 3)


def test_missing_data_and_windows():
    df = D.DataFrame({"v": [1.0, float("nan"), 3.0, float("nan")]})
    assert _col(D.fillna_value(df, "v", 0.0), "v") == [1.0, 0.0, 3.0, 0.0]
    assert _col(D.ffill(df, "v"), "v") == [1.0, 1.0, 3.0, 3.0]
    r = D.rolling_mean_f64([1.0, 2.0, 3.0, 4.0], 2)
    assert (r[0] is None or math.isnan(r[0])) and list(r[1:]) == [1.5, 2.5, 3.5]
    e = D.ewm_mean_f64([1.0, 2.0], 0.5)
    assert abs(e[0] - 1.0) < 1e-12 and 1.0 < e[1] < 2.0


def test_strings_and_io(tmp_path):
    df = D.DataFrame({"s": ["ab", "cd"], "k": [1, 2]})
    assert list(D.str_upper(df, "s")) == ["AB", "CD"]
    p = str(tmp_path / "t.csv")
    D.to_csv(df, p)
    back = D.read_csv(p)
    assert D.df_shape(back) == (2, 2) and _col(back, "s") == ["ab", "cd"]
    j = str(tmp_path / "t.json")
    D.to_json(df, j)
    assert D.df_shape(D.read_json(j)) == (2, 2)


def test_merge_asof():
    left = D.DataFrame({"t": [1, 5, 10], "a": [1, 2, 3]})
    right = D.DataFrame({"t": [2, 3, 7], "b": [10, 20, 30]})
    m = D.merge_asof(left, right, on="t")
    b = _col(m, "b")
    assert (b[0] is None or (isinstance(b[0], float) and math.isnan(b[0]))) and b[1] == 20 and b[2] == 30
