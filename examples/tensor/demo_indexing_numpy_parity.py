"""Selectors on 1-D .. 4-D tensors checked against NumPy, in the spirit of the reference's parity demos
(legacy/examples/tensor/demo_indexing_numpy_parity.mojo, demo_setitem_numpy_parity.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    checks = 0
    a = np.arange(2 * 3 * 4 * 5).reshape(2, 3, 4, 5)
    t = mt.Tensor(a.tolist())
    cases = [
        (lambda x: x[1], "x[1]"), (lambda x: x[:, 1], "x[:, 1]"), (lambda x: x[..., -1], "x[..., -1]"),
        (lambda x: x[0, 1:3, ::2], "x[0, 1:3, ::2]"), (lambda x: x[:, :, ::-1], "x[:, :, ::-1]"),
        (lambda x: x[1, 2, 3, 4], "x[1, 2, 3, 4]"), (lambda x: x[:, [0, 2]], "x[:, [0, 2]]"),
        (lambda x: x[None, 0], "x[None, 0]"),
    ]
    for fn, name in cases:
        got, ref = fn(t), fn(a)
        assert np.array_equal(np.asarray(got.tolist()), ref), name
        checks += 1
    b = a.copy()
    u = mt.Tensor(a.tolist())
    b[0, :, 1] = -1
    u[0, :, 1] = -1
    b[:, 1, ::2, 0] = 7
    u[:, 1, ::2, 0] = 7
    assert np.array_equal(np.asarray(u.tolist()), b)
    checks += 2
    v = mt.arange_f32(0, 12).reshape(3, 4)
    assert np.allclose(np.asarray(mt.math.sum(v, 0).tolist()), np.arange(12, dtype=np.float32).reshape(3, 4).sum(0))
    checks += 1
    print("parity checks passed:", checks)
    return checks


if __name__ == "__main__":
    main()
