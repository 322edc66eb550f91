"""Odds and ends: linspace, eye, tril / triu, diag, cumsum, roll, flip, repeat / tile
(legacy/examples/tensor/demo_misc.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    assert np.allclose(mt.linspace_f64(0.0, 1.0, 5).tolist(), np.linspace(0, 1, 5))
    assert mt.eye_f32(3).tolist() == np.eye(3).tolist()
    a = np.arange(1.0, 10.0).reshape(3, 3)
    t = mt.Tensor(a.tolist())
    assert mt.tril(t).tolist() == np.tril(a).tolist() and mt.triu(t).tolist() == np.triu(a).tolist()
    assert mt.diag(t).tolist() == np.diag(a).tolist()
    assert mt.cumsum(t, 1).tolist() == np.cumsum(a, 1).tolist()
    assert mt.roll(t, 1, 0).tolist() == np.roll(a, 1, 0).tolist()
    assert mt.flip(t, [1]).tolist() == a[:, ::-1].tolist()
    assert mt.tile(t, [1, 2]).tolist() == np.tile(a, (1, 2)).tolist()
    print("misc ok")
    return True


if __name__ == "__main__":
    main()
