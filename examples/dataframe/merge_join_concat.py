"""Inner / left / outer merges, anti join, row and column concatenation
(legacy/examples/dataframe/merge_join_concat.mojo)."""
import momijo.dataframe as D


def main():
    a = D.DataFrame({"k": [1, 2, 3], "x": ["p", "q", "r"]})
    b = D.DataFrame({"k": [2, 3, 4], "y": [20.0, 30.0, 40.0]})
    assert D.merge(a, b, on="k", how="inner").col("k").values == [2, 3]
    left = D.merge(a, b, on="k", how="left")
    assert left.col("k").values == [1, 2, 3] and D.isna(left.col("y").values[0])
    outer = D.merge(a, b, on="k", how="outer")
    assert sorted(outer.col("k").values) == [1, 2, 3, 4]
    anti = D.join_anti(a, b, ["k"], ["k"])
    assert anti.col("k").values == [1]
    rows = D.concat_rows(a, D.DataFrame({"k": [9], "x": ["z"]}))
    assert rows.col("k").values == [1, 2, 3, 9]
    cols = D.concat_cols(a, D.DataFrame({"z": [True, False, True]}))
    assert cols.col_names() == ["k", "x", "z"]
    print(outer.to_string())
    return outer


if __name__ == "__main__":
    main()
