"""Unary and binary element-wise functions, composed, against NumPy
(legacy/examples/tensor/demo_elementwise_custom.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    x = np.linspace(-2.0, 2.0, 17)
    t = mt.Tensor(x.tolist())
    pairs = [(t.exp(), np.exp(x)), (t.abs().sqrt(), np.sqrt(np.abs(x))), (t.tanh(), np.tanh(x)),
             (t.sigmoid(), 1 / (1 + np.exp(-x))), (t.relu(), np.maximum(x, 0)), ((t * t + 1.0).log(), np.log(x * x + 1)),
             (t.sin() * t.cos(), np.sin(x) * np.cos(x)), (mt.clip(t, -1.0, 1.0), np.clip(x, -1, 1))]
    for got, ref in pairs:
        assert np.allclose(np.asarray(got.tolist()), ref, atol=1e-6)
    smooth = lambda v: v * v.sigmoid()          # a user function built from tensor ops (SiLU)
    assert np.allclose(np.asarray(smooth(t).tolist()), x / (1 + np.exp(-x)), atol=1e-6)
    print("element-wise checks:", len(pairs) + 1)
    return len(pairs) + 1


if __name__ == "__main__":
    main()
