"""Pivot table, melt and merge (mirrors legacy/examples/dataframe/pd_pivot_melt_merge.mojo and pivot_reshape.mojo)."""
import momijo.dataframe as D


def main():
    sales = D.DataFrame({"city": ["a", "a", "b", "b"], "year": [2024, 2025, 2024, 2025], "amount": [1.0, 2.0, 3.0, 4.0]})
    wide = sales.pivot_table("city", "year", "amount", "sum")
    long = wide.melt(["city"], "year", "amount")
    regions = D.DataFrame({"city": ["a", "b"], "region": ["north", "south"]})
    joined = long.merge(regions, "city", "left")
    print(wide.to_string(), long.to_string(), joined.to_string(), sep="\n")
    assert joined.nrows() == 4 and joined.has_col("region")
    return joined


if __name__ == "__main__":
    main()
