"""CSV and JSON round trips through strings and files (mirrors legacy/examples/dataframe/io_csv_json.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"id": [1, 2], "label": ["a,b", 'say "hi"']})
    csv_text = D.to_csv_string(df)
    back = D.read_csv_from_string(csv_text)
    json_text = D.to_json_string(df)
    back_json = D.from_json_string(json_text)
    assert df.to_csv("frame.csv") and D.read_csv("frame.csv").nrows() == 2
    print(csv_text, json_text, sep="\n")
    assert back.col("label").values == df.col("label").values == back_json.col("label").values
    return back


if __name__ == "__main__":
    main()
