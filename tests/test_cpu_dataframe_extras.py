"""Window statistics, joins, plans, parsers and text I/O of the dataframe package."""
import math

import momijo_b200.dataframe as D


def test_window_statistics():
    assert D.rolling_var_f64([1, 2, 3, 4], 2, 1) == [None, 0.5, 0.5, 0.5]
    assert D.rolling_std_f64([1, 2, 3, 4], 2) == [None, 0.5, 0.5, 0.5]
    assert D.rolling_sum_int([1, 2, 3], 2) == [None, 3, 5] and D.rolling_max_f64([1, 3, 2], 2) == [None, 3, 3]
    assert D.ewm_mean_f64([1.0, 2.0], 0.5) == [1.0, 1.5]
    adj = D.ewm_mean_f64([1, 2, 3], 0.5, True)
    assert abs(adj[2] - (0.25 * 1 + 0.5 * 2 + 1 * 3) / 1.75) < 1e-12
    assert D.ewm_var_f64([1, 2, 3], 0.5) == [0.0, 0.25, 0.6875] and D.ewm_mean_f64([1], 1.5) == []
    v = D.expanding_var_f64([1, 2, 3], 1)
    assert math.isnan(v[0]) and abs(v[2] - 1.0) < 1e-9
    assert D.expanding_mean_f64([2, 4], 2)[1] == 3.0 and math.isnan(D.expanding_mean_f64([2, 4], 2)[0])
    assert D.lag([1, 2, 3]) == [None, 1, 2] and D.lead([1, 2, 3], 2) == [3, None, None]
    assert D.rank_dense_f64([3.0, 1.0, 3.0, 2.0]) == [3, 1, 3, 2] and D.percentile_f64([1, 2, 3, 4], 50) == 2.5
    assert D.nlargest_f64([1, 5, 3], 2) == [1, 2] and D.argsort_f64([3, 1, 2], False) == [0, 2, 1]
    assert abs(D.corr([1, 2, 3], [2, 4, 6]) - 1.0) < 1e-12 and D.corr([1, 1], [1, 2]) == 0.0


def test_joins_and_groupby():
    L = D.DataFrame({"k": [1, 2, 3], "a": ["x", "y", "z"]})
    R = D.DataFrame({"k": [2, 3, 3, 4], "b": [20, 30, 31, 40]})
    assert [r["b"] for r in D.join_inner(L, R, ["k"], ["k"]).to_records()] == [20, 30, 31]
    assert D.join_left(L, R, ["k"], ["k"]).nrows() == 4 and D.join_right(L, R, ["k"], ["k"]).nrows() == 4
    assert D.join_full(L, R, ["k"], ["k"]).to_records()[-1] == {"k": 4, "a": None, "b": 40}
    assert D.join_anti(L, R, ["k"], ["k"]).to_records() == [{"k": 1, "a": "x"}]
    asof = D.asof_join(D.DataFrame({"t": [1, 5, 10]}), D.DataFrame({"t": [2, 6], "v": [20, 60]}), "t")
    assert asof.col("v").values == [None, 20, 60]
    df = D.DataFrame({"g": ["a", "b", "a"], "x": [1.0, 2.0, 3.0], "s": ["p", "q", "r"]})
    assert D.groupby_agg(df, ["g"], [("x", "sum"), ("x", "mean")]).to_records()[0] == {"g": "a", "x_sum": 4.0, "x_mean": 2.0}
    assert D.groupby_sum_f64(df, "g", "x").col("x").values == [4.0, 2.0] and D.apply_agg([1, None, 3], "mean") == 2.0
    assert D.exec_aggregate(df, [], [D.AggSpec("x", "count", "n")]).to_records() == [{"n": 3.0}]
    assert D.eval_where(df, "x >= 2 and g == 'a' or s == 'p'").bits == [True, False, True]
    P = D.relational
    plan = D.LogicalPlan(P.PLAN_FILTER, expr=D.parse_simple_expr("g == 'a'"),
                         child=D.LogicalPlan(P.PLAN_FILTER, child=D.LogicalPlan(df=df), expr=D.parse_simple_expr("x > 1")))
    opt = D.optimize(plan)
    assert opt.child.kind == P.PLAN_SCAN and D.execute(opt).to_records() == [{"g": "a", "x": 3.0, "s": "r"}]
    assert D.query(df, "y = 2 * x").col("y").values == [2.0, 4.0, 6.0] and D.eval(df, "nonsense") is df


def test_resample_categorical_series():
    ts = D.DataFrame({"v": [1, 2, 3, 4]}, index=["2025-01-01", "2025-01-02 10:00:00", "2025-01-03", "2025-01-05"])
    r = D.resample(ts, "2D").sum()
    assert r.col("v").values == [3.0, 3.0, 4.0] and list(r.index.labels) == ["2025-01-01", "2025-01-03", "2025-01-05"]
    assert D.gen_dates_12h_from_2025_01_01(2) == ["2025-01-01 00:00:00", "2025-01-01 12:00:00"]
    assert D.parse_minutes("2025-01-01 10:30:00") == 630 and D.tz_localize_utc(["t"]) == ["t+00:00"]
    c = D.Categorical(["a", "b", "a", None])
    assert c.codes_list() == [0, 1, 0, -1] and c.value_counts() == {"a": 2, "b": 1}
    assert c.reorder(["b"]).values() == ["", "b", "", ""] and D.Categorical(["x"], ["x", "y"]).remove_unused().categories() == ["x"]
    assert D.SeriesF64([1, None, 3]).mean() == 2.0 and D.SeriesStr([1]).get(0) == "1"
    assert D.resolve_label_slice(["a", "b", "c"], D.LabelSlice("a", "b")) == [0, 1]


def test_parsers_helpers_and_text_io():
    df = D.DataFrame({"city": ["a", "b", "a"], "qty": [1, 5, 3], "x": [1.5, None, 2.5]})
    for back in (D.from_mnp_string(D.to_mnp_string(df)), D.from_json_string(D.to_json_string(df)),
                 D.from_json_lines_string(D.to_json_lines_string(df)), D.read_csv_from_string(D.to_csv_string(df))):
        assert D.equals(df, back)
    tricky = D.DataFrame({"s": ["tab\there", "line\nbreak", "back\\slash"]})
    assert D.equals(tricky, D.from_mnp_string(D.to_mnp_string(tricky)))
    assert D.df_nlargest(df, "qty", 2).col("qty").values == [5, 3] and D.df_where_qty_between(df, 2, 5).nrows() == 2
    assert D.get_dummies_str(df, "city").col_names() == ["qty", "x", "city_a", "city_b"]
    assert D.value_counts_str(["a", "b", "a"]).to_records()[0] == {"value": "a", "count": 2}
    assert D.as_i64_or_zero("3.9") == 3 and D.as_f64_or_nan("1,5") == 1.5 and D.as_bool_or_false(" Yes ")
    assert D.infer_dtype(["1", "2"]) == "int" and D.infer_dtype(["1", "x"]) == "string" and D.infer_dtype(["1.5"]) == "float"
    assert D.split_on_delims("a, b;c|d") == ["a", "b", "c", "d"] and D.str_split_once("k=v=w", "=") == ("k", "v=w")
    assert D.atoi("-12ab") == -12 and D.symdiff(["a", "b"], ["b", "c"]) == ["a", "c"]
    assert D.tag_name(D.dtype_to_tag(D.float64)) == "float64" and D.is_f64_col(df.col("x")) and D.is_str_col(df.col("city"))
    a, b = D.align_columns(df, D.DataFrame({"z": [1]}))
    assert a.col_names() == b.col_names() == ["city", "qty", "x", "z"] and b.col("city").values == [None]
    assert D.col_f64("c", [1.0, 2.0], D.make_bitmap(2, False)).values == [None, None]
    assert D.dropna_rows(df).nrows() == 2 and D.range(3) == [0, 1, 2]
