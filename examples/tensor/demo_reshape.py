"""reshape / view / flatten / squeeze / unsqueeze and inferred dimensions
(legacy/examples/tensor/demo_reshape.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = np.arange(24.0)
    t = mt.Tensor(a.tolist())
    r = mt.reshape(t, [2, 3, 4])
    assert r.tolist() == a.reshape(2, 3, 4).tolist()
    assert list(mt.reshape_infer(t, [4, -1]).shape) == [4, 6]
    assert mt.flatten(r).tolist() == a.tolist()
    u = mt.unsqueeze(r, 1)
    assert list(u.shape) == [2, 1, 3, 4] and list(mt.squeeze(u).shape) == [2, 3, 4]
    assert list(mt.view(t, [6, 4]).shape) == [6, 4]
    assert mt.transpose(mt.reshape(t, [4, 6]), 0, 1).tolist() == a.reshape(4, 6).T.tolist()
    print("reshape ok")
    return True


if __name__ == "__main__":
    main()
