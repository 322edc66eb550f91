"""assign with constants, lists and functions of the frame; chained with pipe
(legacy/examples/dataframe/dataframe_setitem_assign.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"qty": [2, 5, 1], "price": [3.0, 1.5, 10.0]})
    out = df.assign({"total": lambda d: [q * p for q, p in zip(d.col("qty").values, d.col("price").values)],
                     "flag": [True, False, True], "unit": "eur"})
    assert out.col("total").values == [6.0, 7.5, 10.0] and out.col("unit").values == ["eur"] * 3
    assert df.col_names() == ["qty", "price"]          # assign returns a new frame
    big = out.pipe(lambda d: D.filter_rows(d, [t > 6.5 for t in d.col("total").values]))
    assert big.col("qty").values == [5, 1]
    print(big.to_string())
    return big


if __name__ == "__main__":
    main()
