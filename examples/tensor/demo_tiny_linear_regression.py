"""Least squares by gradient descent with the autograd tape
(legacy/examples/tensor/demo_tiny_linear_regression.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    rng = np.random.default_rng(2)
    x = rng.normal(size=(64, 3))
    w_true = np.array([[1.5], [-2.0], [0.5]])
    y = x @ w_true + 0.3
    X, Y = mt.Tensor(x.tolist()), mt.Tensor(y.tolist())
    w = mt.zeros_f64([3, 1]).requires_grad_(True)
    b = mt.zeros_f64([1]).requires_grad_(True)
    losses = []
    for _ in range(200):
        loss = ((mt.matmul(X, w) + b - Y) ** 2).mean()
        loss.backward()
        with mt.torch.no_grad():
            w -= 0.1 * w.grad
            b -= 0.1 * b.grad
        w.grad = None
        b.grad = None
        losses.append(loss.item())
    assert losses[-1] < 1e-6 and np.allclose(w.tolist(), w_true, atol=1e-3) and abs(b.item() - 0.3) < 1e-3
    print("fitted", [round(v[0], 3) for v in w.tolist()], round(b.item(), 3))
    return losses[-1]


if __name__ == "__main__":
    main()
