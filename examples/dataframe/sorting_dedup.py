"""Sorting, dense ranks and duplicate removal (mirrors legacy/examples/dataframe/sorting_dedup.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"name": ["x", "y", "x", "z"], "score": [3, 1, 3, 2]})
    ordered = D.sort_values(df, "score", ascending=False)
    unique_first = df.drop_duplicates()
    unique_last = df.drop_duplicates(["name"], "last")
    print(ordered.to_string(), unique_first.to_string(), unique_last.to_string(), sep="\n")
    print("dense rank:", D.dense_rank(df.col("score").values))
    assert unique_first.nrows() == 3 and unique_last.index.labels == [1, 2, 3]
    return ordered


if __name__ == "__main__":
    main()
