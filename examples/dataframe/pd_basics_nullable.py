"""Missing values: nullable construction, isna counts, fill and drop
(legacy/examples/dataframe/pd_basics_nullable.mojo)."""
import momijo.dataframe as D


def main():
    df = D.ToDataFrameNullable({"a": ["1", "", "3"], "b": ["x", "y", ""]}, null_token="")
    counts = D.isna_count_by_col(df)
    print(counts)
    filled = D.fillna_value(df, "b", "?")
    assert filled.col("b").values[2] == "?"
    kept = D.dropna_any(df)
    assert kept.nrows() == 1
    num = D.DataFrame({"x": [1.0, float("nan"), float("nan"), 4.0]})
    assert D.ffill(num, "x").col("x").values == [1.0, 1.0, 1.0, 4.0]
    interp = D.interpolate_numeric(D.DataFrame({"x": [1.0, float("nan"), 3.0]}), "x")
    assert interp.col("x").values == [1.0, 2.0, 3.0]
    print(kept.to_string())
    return kept


if __name__ == "__main__":
    main()
