"""A method chain: assign -> filter -> group-by -> sort
(legacy/examples/dataframe/pd_assign_pipe_groupby.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"shop": ["n", "s", "n", "s", "n"], "qty": [3, 1, 4, 1, 5], "price": [2.0, 7.0, 1.0, 8.0, 2.0]})
    out = (df.assign({"rev": lambda d: [q * p for q, p in zip(d.col("qty").values, d.col("price").values)]})
             .pipe(lambda d: D.filter_rows(d, [r >= 4.0 for r in d.col("rev").values]))
             .pipe(lambda d: D.groupby(d, "shop", [D.Agg("rev", "sum", "rev_sum"), D.Agg("qty", "max", "qty_max")]))
             .sort_values("rev_sum", ascending=False))
    assert out.col("shop").values == ["n", "s"] and out.col("rev_sum").values == [20.0, 15.0]
    print(out.to_string())
    return out


if __name__ == "__main__":
    main()
