"""Column dtypes, casts, date ranges and year extraction
(legacy/examples/dataframe/dtypes_datetime.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"i": [1, 2, 3], "f": [1.5, 2.5, 3.5], "s": ["x", "y", "z"], "b": [True, False, True]})
    print(D.df_dtypes(df))
    as_f = D.astype(df, "i", "float64")
    assert as_f.col("i").values == [1.0, 2.0, 3.0]
    dates = D.date_range("2025-01-30", 4)
    assert dates[0].startswith("2025-01-30") and dates[2].startswith("2025-02-01")
    years = D.datetime_year(["2024-12-31", "2025-01-01"])
    assert list(years) == [2024, 2025]
    half_days = D.gen_dates_12h_from_2025_01_01(3)
    assert len(half_days) == 3
    print(dates, list(years))
    return dates


if __name__ == "__main__":
    main()
