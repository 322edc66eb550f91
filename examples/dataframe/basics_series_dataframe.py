"""Series and DataFrame construction, shape, columns, head / tail, describe
(legacy/examples/dataframe/basics_series_dataframe.mojo)."""
import momijo.dataframe as D


def main():
    s = D.series_from_list([3, 1, 2], "n")
    assert list(s.values) == [3, 1, 2] and s.name == "n"
    df = D.DataFrame({"name": ["ann", "bob", "cy", "di"], "age": [31, 25, 47, 19], "score": [1.5, 2.5, 3.0, 4.0]})
    assert df.shape() == (4, 3) and df.col_names() == ["name", "age", "score"]
    assert df.head(2).col("name").values == ["ann", "bob"] and df.tail(1).col("age").values == [19]
    assert df.col("age").values[2] == 47 and df.row(1)["name"] == "bob"
    print(df.to_string())
    print(df.describe().to_string() if hasattr(df.describe(), "to_string") else df.describe())
    return df


if __name__ == "__main__":
    main()
