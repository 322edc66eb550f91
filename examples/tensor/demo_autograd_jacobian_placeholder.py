"""Jacobian of a small vector function, row by row, from the autograd tape
(legacy/examples/tensor/demo_autograd_jacobian_placeholder.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    x = mt.Tensor([1.0, 2.0, 3.0]).double().requires_grad_(True)
    def f(v):
        return mt.stack([v[0] * v[1], v[1] ** 2 + v[2], v.sum() * v[0]])
    y = f(x)
    rows = []
    for i in range(3):
        g, = mt.torch.autograd.grad(y[i], x, retain_graph=True)
        rows.append(g.tolist())
    ref = [[2.0, 1.0, 0.0], [0.0, 4.0, 1.0], [7.0, 1.0, 1.0]]
    assert np.allclose(rows, ref)
    print("jacobian", rows)
    return rows


if __name__ == "__main__":
    main()
