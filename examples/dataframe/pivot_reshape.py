"""pivot_table, melt and back, dummies
(legacy/examples/dataframe/pivot_reshape.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"day": ["mon", "mon", "tue", "tue"], "shop": ["n", "s", "n", "s"], "v": [1.0, 2.0, 3.0, 4.0]})
    wide = df.pivot_table("day", "shop", "v", aggfunc="sum")
    assert wide.col("day").values == ["mon", "tue"] and wide.col("n").values == [1.0, 3.0] and wide.col("s").values == [2.0, 4.0]
    long = wide.melt(["day"], var_name="shop", value_name="v")
    assert long.nrows() == 4 and sorted(long.col("v").values) == [1.0, 2.0, 3.0, 4.0]
    dum = D.get_dummies_str(df, "shop")
    assert any(c.endswith("n") for c in dum.col_names()) and any(c.endswith("s") for c in dum.col_names())
    print(wide.to_string())
    print(long.to_string())
    return wide


if __name__ == "__main__":
    main()
