"""moveaxis / swapaxes, sliding windows, cumulative ops and quantiles along an axis
(legacy/examples/tensor/demo_tensor_axis_windows.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = np.arange(24.0).reshape(2, 3, 4)
    t = mt.Tensor(a.tolist())
    assert mt.moveaxis(t, 0, 2).tolist() == np.moveaxis(a, 0, 2).tolist()
    assert mt.swapaxes(t, 1, 2).tolist() == np.swapaxes(a, 1, 2).tolist()
    w = mt.sliding_window(mt.Tensor(list(range(6))), 3)
    assert w.tolist() == [[0, 1, 2], [1, 2, 3], [2, 3, 4], [3, 4, 5]]
    assert mt.cumprod(mt.Tensor([1.0, 2.0, 3.0]), 0).tolist() == [1.0, 2.0, 6.0]
    assert np.allclose(mt.median(t, 2).tolist(), np.median(a, 2))
    assert np.allclose(mt.quantile(t, 0.25, 2).tolist(), np.quantile(a, 0.25, 2))
    print("axis / window ops ok")
    return True


if __name__ == "__main__":
    main()
