"""Row and column selection: loc / iloc call forms, masks and query strings
(mirrors legacy/examples/dataframe/selection_filtering.mojo and dataframe_indexing.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"city": ["a", "b", "c", "d"], "qty": [5, 12, 7, 20], "ok": [True, False, True, True]})
    head2 = df.iloc([0, 1], D.ColAll())
    qty = df.iloc(D.RowAll(), 1)
    big = D.filter_rows(df, D.eval_where(df, "qty >= 7 and city != 'b'").to_mask())
    scaled = D.query(df, "double = qty * 2")
    masked = D.filter_rows(df, D.mask_and([q > 5 for q in df.col("qty").values], df.col("ok").values))
    cell = df.at(2, "city").get()
    print(head2.to_string(), big.to_string(), masked.to_string(), sep="\n")
    assert qty.to_list() == [5, 12, 7, 20] and cell == "c" and scaled.col("double").values[1] == 24.0 and big.col("city").values == ["c", "d"] == masked.col("city").values
    return big


if __name__ == "__main__":
    main()
