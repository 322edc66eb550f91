"""Right-aligned broadcasting of shapes and binary ops
(legacy/examples/tensor/demo_broadcast_align.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    assert mt.broadcast_shapes([3, 1, 5], [4, 1]) == [3, 4, 5]
    a = mt.Tensor(np.arange(15.0).reshape(3, 1, 5).tolist())
    b = mt.Tensor(np.arange(4.0).reshape(4, 1).tolist())
    c = a + b
    ref = np.arange(15.0).reshape(3, 1, 5) + np.arange(4.0).reshape(4, 1)
    assert tuple(c.shape) == (3, 4, 5) and np.array_equal(np.asarray(c.tolist()), ref)
    e = mt.broadcast_to(b, [2, 4, 3])
    assert tuple(e.shape) == (2, 4, 3) and np.array_equal(np.asarray(e.tolist()), np.broadcast_to(np.arange(4.0).reshape(4, 1), (2, 4, 3)))
    s = a * 2.0 - 1.0
    assert np.array_equal(np.asarray(s.tolist()), np.arange(15.0).reshape(3, 1, 5) * 2 - 1)
    print("broadcast shape", list(c.shape))
    return list(c.shape)


if __name__ == "__main__":
    main()
