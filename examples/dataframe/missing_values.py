"""Counting, filling and dropping missing cells (mirrors legacy/examples/dataframe/missing_values.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"qty": [1.0, None, 3.0, None], "city": ["a", None, "c", "d"]})
    print("missing per column:", D.isna_count_by_col(df))
    filled = D.fillna_value(df, "qty", 0.0)
    carried = D.ffill(df, "qty")
    complete = D.dropna_rows(df)
    print(filled.to_string(), carried.to_string(), complete.to_string(), sep="\n")
    assert complete.nrows() == 2 and df.col("qty").null_count() == 2
    return complete


if __name__ == "__main__":
    main()
