"""Sums, means, variance, quantiles, cumulative ops and NaN-aware reductions
(mirrors legacy/examples/tensor/demo_reductions_stats.mojo, demo_tensor_stats.mojo and demo_masked_reductions.mojo)."""
import momijo.tensor as mt


def main():
    x = mt.from_list([[1.0, 2.0, 3.0], [4.0, float("nan"), 6.0]])
    clean = mt.nanops.nan_to_num(x, nan=0.0)
    print("sum by row:", mt.math.sum(clean, 1).tolist(), "mean by column:", mt.mean(clean, 0).tolist())
    print("nan-aware sum:", mt.nanops.nansum(x, 1).tolist(), "nan-aware mean:", x.nanmean(1).tolist())
    print("cumsum:", mt.cumsum(clean, 1).tolist(), "median:", mt.median(clean).item())
    print("quantile 0.25:", mt.quantile(clean.flatten_all(), 0.25).item(), "argmax:", mt.math.argmax(clean).item())
    assert mt.nanops.nansum(x, 1).tolist() == [6.0, 10.0] and mt.axis.nanargmax(x, axis=1).tolist() == [2, 2]
    assert abs(float(mt.math.var(clean, unbiased=False)) - float(clean.var_all())) < 1e-6
    return clean


if __name__ == "__main__":
    main()
