"""softmax / log-softmax / logsumexp on large logits stay finite
(legacy/examples/tensor/demo_numerical_stability.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    x = np.array([[1000.0, 1001.0, 999.0], [-1000.0, -999.0, -1001.0]])
    t = mt.Tensor(x.tolist())
    p = mt.softmax(t)
    ref = np.exp(x - x.max(1, keepdims=True))
    ref /= ref.sum(1, keepdims=True)
    assert np.allclose(np.asarray(p.tolist()), ref) and np.isfinite(np.asarray(p.tolist())).all()
    lp = mt.log_softmax(t)
    assert np.allclose(np.asarray(lp.tolist()), np.log(ref))
    lse = t.logsumexp(1)
    assert np.allclose(np.asarray(lse.tolist()), x.max(1) + np.log(np.exp(x - x.max(1, keepdims=True)).sum(1)))
    assert mt.nanops.safe_div(mt.Tensor([1.0, 2.0]), mt.Tensor([0.0, 4.0])).tolist()[1] == 0.5
    print("stable softmax rows sum to", p.sum(1).tolist())
    return True


if __name__ == "__main__":
    main()
