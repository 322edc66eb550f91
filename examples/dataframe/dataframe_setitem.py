"""Cell, column and row assignment
(legacy/examples/dataframe/dataframe_setitem.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"a": [1, 2, 3], "b": [1.0, 2.0, 3.0]})
    assert df.set_iat(0, 0, 9) and df.col("a").values[0] == 9
    df.set_column("c", [True, False, True])
    assert df.col_names() == ["a", "b", "c"] and df.col("c").values == [True, False, True]
    df.set_column("b", [x * 10 for x in df.col("b").values])
    assert df.col("b").values == [10.0, 20.0, 30.0]
    df2 = D.set_value(df, 2, "a", -1)
    assert df2.col("a").values[2] == -1
    df3 = df2.drop(["c"])
    assert df3.col_names() == ["a", "b"]
    print(df3.to_string())
    return df3


if __name__ == "__main__":
    main()
