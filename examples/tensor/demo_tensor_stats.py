"""mean / var / std / min / max / argmax along axes, percentiles
(legacy/examples/tensor/demo_tensor_stats.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    rng = np.random.default_rng(1)
    a = rng.normal(size=(5, 7))
    t = mt.Tensor(a.tolist())
    assert np.allclose(t.mean(0).tolist(), a.mean(0)) and np.allclose(t.mean().item(), a.mean())
    assert np.allclose(t.var(1, unbiased=False).tolist(), a.var(1)) and np.allclose(t.std(1).tolist(), a.std(1, ddof=1))
    assert t.argmax(1).tolist() == a.argmax(1).tolist() and t.argmin(0).tolist() == a.argmin(0).tolist()
    assert np.allclose(t.max().item(), a.max()) and np.allclose(t.min(1).values.tolist(), a.min(1))
    assert np.allclose(mt.percentile(t, 90.0, 1).tolist(), np.percentile(a, 90, 1))
    assert np.allclose(mt.mean(t, 1).tolist(), a.mean(1))
    print("stats ok")
    return True


if __name__ == "__main__":
    main()
