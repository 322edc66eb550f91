"""Rolling, expanding and exponentially weighted statistics over a price list
(mirrors legacy/examples/dataframe/pd_rolling_expanding_ewm.mojo)."""
import momijo.dataframe as D


def main():
    prices = [10.0, 10.5, 10.2, 11.0, 11.4, 11.1]
    out = D.DataFrame({
        "price": prices,
        "roll_mean_3": D.rolling_mean_f64(prices, 3),
        "roll_sum_3": D.rolling_sum_f64(prices, 3),
        "roll_std_3": D.rolling_std_f64(prices, 3),
        "exp_mean": D.expanding_mean_f64(prices),
        "ewm_alpha": D.ewm_mean_f64(prices, 0.5),
        "ewm_span": D.ewm_mean_f64_span(prices, 3),
    })
    print(out.to_string())
    return out


if __name__ == "__main__":
    main()
