"""Multi-level index, as-of join and a JSON-lines round trip
(mirrors legacy/examples/dataframe/pd_multiindex_asof_io.mojo)."""
import momijo.dataframe as D


def main():
    mi = D.MultiIndex.from_product([["a", "b"], ["x", "y"]], ["outer", "inner"])
    print("levels:", mi.levels_copy(), "codes:", mi.codes_copy(), "sorted:", mi.is_lexsorted())
    quotes = D.DataFrame({"t": [1, 5, 10], "bid": [100.0, 101.0, 102.0]})
    trades = D.DataFrame({"t": [2, 6, 11], "size": [10, 20, 30]})
    joined = D.asof_join(trades, quotes, "t")
    lines = D.to_json_lines_string(joined)
    back = D.from_json_lines_string(lines)
    print(joined.to_string(), lines, sep="\n")
    assert mi.nrows() == 4 and back.nrows() == 3 and joined.col("bid").values == [100.0, 101.0, 102.0]
    return joined


if __name__ == "__main__":
    main()
