"""Whole-column arithmetic without Python-level row loops: cumulative sums, lags, ranks, rolling windows
(legacy/examples/dataframe/vectorize_demo.mojo)."""
import momijo.dataframe as D


def main():
    xs = [3.0, 1.0, 4.0, 1.0, 5.0, 9.0]
    assert D.cum_sum(xs) == [3.0, 4.0, 8.0, 9.0, 14.0, 23.0]
    assert D.lag(xs, 1, fill=0.0) == [0.0, 3.0, 1.0, 4.0, 1.0, 5.0]
    assert D.rolling_mean_f64(xs, 2)[1:] == [2.0, 2.5, 2.5, 3.0, 7.0]
    assert D.rank_dense_f64(xs) == [2, 1, 3, 1, 4, 5]
    assert D.nlargest_f64(xs, 2) == [5, 4]
    df = D.DataFrame({"x": xs})
    t = df.to_tensor()
    assert abs(float(t.sum()) - 23.0) < 1e-9          # hand the column block to the tensor engine
    clipped = D.clip_f64(xs, 2.0, 5.0)
    assert clipped == [3.0, 2.0, 4.0, 2.0, 5.0, 5.0]
    print(D.cum_sum(xs), clipped)
    return clipped


if __name__ == "__main__":
    main()
