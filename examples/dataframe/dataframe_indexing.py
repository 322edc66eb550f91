"""loc / iloc / at / iat call forms with labels, positions and ranges
(legacy/examples/dataframe/dataframe_indexing.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"k": ["a", "b", "c", "d"], "x": [10, 20, 30, 40], "y": [0.1, 0.2, 0.3, 0.4]})
    df = D.df_set_index(df, "k")
    assert df.iloc([0, 2], D.ColAll()).col("x").values == [10, 30]
    assert df.iloc(D.RowAll(), 0).to_list() == [10, 20, 30, 40]
    assert df.loc(["b", "d"], ["y"]).col("y").values == [0.2, 0.4]
    assert df.at("c", "x").col("x").values == [30] and df.iat(3, 1).col("y").values == [0.4]   # one-cell frames
    sub = df.iloc([1, 2], D.ColAll())
    assert sub.col("x").values == [20, 30]
    print(sub.to_string())
    return sub


if __name__ == "__main__":
    main()
