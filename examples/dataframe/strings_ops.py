"""String columns: case, length, contains, replace, slices, splits
(legacy/examples/dataframe/strings_ops.mojo)."""
import momijo.dataframe as D


def main():
    df = D.DataFrame({"s": ["  Maple ", "oak", "Red maple", "pine"]})
    up = D.str_upper(df, "s")
    vals = up.col("s").values if hasattr(up, "col") else list(up)
    assert vals[1] == "OAK"
    assert D.str_len(df, "s") == [8.0, 3.0, 9.0, 4.0]
    has = D.str_contains(df, "s", "maple", case_insensitive=True)
    mask = has.to_mask() if hasattr(has, "to_mask") else list(has)
    assert list(mask) == [True, False, True, False]
    assert D.str_strip("  Maple ") == "Maple"
    titled = D.str_title(df, "s")
    assert (titled.col("s").values if hasattr(titled, "col") else list(titled))[2].strip() == "Red Maple"
    assert D.str_replace_all("a-b-c", "-", "+") == "a+b+c"
    sl = D.str_slice(df, "s", 0, 3)
    assert (sl.col("s").values if hasattr(sl, "col") else list(sl))[1] == "oak"
    assert tuple(D.str_split_once("key=value", "=")) == ("key", "value")
    print(vals, list(mask))
    return vals


if __name__ == "__main__":
    main()
