"""Group-by, merge and rolling statistics on a small frame (the reference ships 22 such demos under
legacy/examples/dataframe/)."""
import momijo.dataframe as D


def main():
    sales = D.DataFrame({"city": ["a", "b", "a", "c", "b", "a"], "amount": [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]})
    pop = D.DataFrame({"city": ["a", "b", "c"], "pop": [10, 20, 30]})
    by_city = D.groupby(sales, "city", [D.Agg("amount", "sum", "total"), D.Agg("amount", "count", "n")])
    joined = D.merge(by_city, pop, on="city", how="left")
    print(joined)
    print("rolling mean:", D.rolling_mean_f64([1.0, 2.0, 3.0, 4.0], 2))
    return joined


if __name__ == "__main__":
    main()
