"""CSV / JSON / JSON-lines / MNP text round trips in memory and on disk
(legacy/examples/dataframe/io.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"id": [1, 2, 3], "name": ["a,b", "c", "d"], "v": [0.5, 1.5, 2.5]})
    csv = D.to_csv_string(df)
    back = D.read_csv_from_string(csv)
    assert back.col("name").values == ["a,b", "c", "d"] and back.col("v").values == [0.5, 1.5, 2.5]
    js = D.to_json_string(df)
    assert D.from_json_string(js).col("id").values == [1, 2, 3]
    jl = D.to_json_lines_string(df)
    assert D.from_json_lines_string(jl).col("name").values == ["a,b", "c", "d"]
    mnp = D.to_mnp_string(df)
    assert D.from_mnp_string(mnp).col("v").values == [0.5, 1.5, 2.5]
    assert df.to_csv("frame.csv", index=False)
    assert D.read_csv("frame.csv").col("id").values == [1, 2, 3]
    print(csv)
    return back


if __name__ == "__main__":
    main()
