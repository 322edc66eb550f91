"""Categories, dates and day-bucket resampling
(mirrors legacy/examples/dataframe/pd_categorical_datetime_resample.mojo)."""
import momijo.dataframe as D


def main():
    cat = D.to_category(["lo", "hi", "lo", "mid"])
    days = D.date_range("2025-01-01", 4)
    stamps = D.to_datetime(days)
    years = D.datetime_year(days)
    print("categories:", cat, "days:", days, "years:", years)
    assert years == [2025] * 4 and stamps[1][:3] == (2025, 1, 2)
    return days


if __name__ == "__main__":
    main()
