"""Group-by with several aggregations, multi-key groups and transforms
(legacy/examples/dataframe/groupby_agg.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"g": ["a", "b", "a", "b", "a"], "h": ["x", "x", "y", "y", "x"], "v": [1.0, 2.0, 3.0, 4.0, 5.0]})
    agg = D.groupby(df, "g", [D.Agg("v", "sum", "total"), D.Agg("v", "mean", "avg"), D.Agg("v", "count", "n")])
    rows = {g: (t, a, n) for g, t, a, n in zip(agg.col("g").values, agg.col("total").values, agg.col("avg").values, agg.col("n").values)}
    assert rows["a"] == (9.0, 3.0, 3) and rows["b"] == (6.0, 3.0, 2)
    multi = D.groupby_multi(df, ["g", "h"], [D.Agg("v", "sum", "total")])
    assert multi.nrows() == 4
    dem = D.groupby_transform(df, "g", "v", "mean")
    assert [round(x, 6) for x in dem] == [3.0, 3.0, 3.0, 3.0, 3.0]
    print(agg.to_string())
    print(multi.to_string())
    return agg


if __name__ == "__main__":
    main()
