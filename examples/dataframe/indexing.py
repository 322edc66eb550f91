"""Boolean masks, isin, between and position slices
(legacy/examples/dataframe/indexing.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"city": ["a", "b", "c", "d", "e"], "qty": [5, 12, 7, 20, 1]})
    m1 = D.filter_rows(df, [q > 6 for q in df.col("qty").values])
    assert m1.col("city").values == ["b", "c", "d"]
    m2 = D.filter_rows(df, [D.isin_string(c, ["a", "e"]) for c in df.col("city").values])
    assert m2.col("qty").values == [5, 1]
    m3 = D.filter_rows(df, [D.between_i64(q, 5, 12) for q in df.col("qty").values])
    assert m3.col("city").values == ["a", "b", "c"]
    top = D.slice_rows(D.sort_values(df, "qty", ascending=False), 0, 2)
    assert top.col("city").values == ["d", "b"]
    print(top.to_string())
    return top


if __name__ == "__main__":
    main()
